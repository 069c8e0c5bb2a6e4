"""The PyTorch oracles themselves are checked against autograd / torch.nn so GPU kernels are compared to something sound."""
import math

import torch

from nanotron_b200 import ops
from nanotron_b200.ops import reference as ref


def test_rms_norm_backward_matches_autograd():
    torch.manual_seed(0)
    x = torch.randn(6, 32, dtype=torch.float64, requires_grad=True)
    r = torch.randn(6, 32, dtype=torch.float64, requires_grad=True)
    w = torch.randn(32, dtype=torch.float64, requires_grad=True)
    y, pre = ops.rms_norm(x, w, 1e-5, residual=r)
    (y.sum() + (pre * 2).sum()).backward()
    x2, r2, w2 = (t.detach().clone().requires_grad_(True) for t in (x, r, w))
    pre2 = x2 + r2
    y2 = pre2 * torch.rsqrt(pre2.pow(2).mean(-1, keepdim=True) + 1e-5) * w2
    (y2.sum() + (pre2 * 2).sum()).backward()
    torch.testing.assert_close(x.grad, x2.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(r.grad, r2.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(w.grad, w2.grad, atol=1e-4, rtol=1e-4)


def test_layer_norm_matches_torch():
    torch.manual_seed(1)
    x = torch.randn(5, 16, dtype=torch.float64, requires_grad=True)
    w = torch.randn(16, dtype=torch.float64, requires_grad=True)
    b = torch.randn(16, dtype=torch.float64, requires_grad=True)
    y = ops.layer_norm(x, w, b, 1e-5)
    y.pow(2).sum().backward()
    x2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    torch.nn.functional.layer_norm(x2, (16,), w2, b2, 1e-5).pow(2).sum().backward()
    torch.testing.assert_close(x.grad, x2.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(w.grad, w2.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(b.grad, b2.grad, atol=1e-4, rtol=1e-4)


def test_swiglu_backward_matches_autograd():
    gu = torch.randn(4, 16, dtype=torch.float64, requires_grad=True)
    ops.swiglu(gu).sum().backward()
    g2 = gu.detach().clone().requires_grad_(True)
    a, b = g2.chunk(2, -1)
    (torch.nn.functional.silu(a) * b).sum().backward()
    torch.testing.assert_close(gu.grad, g2.grad, atol=1e-4, rtol=1e-4)


def test_rope_inverse_is_transpose():
    x = torch.randn(7, 2, 8, dtype=torch.float64)
    cos, sin = ref.rope_cos_sin(torch.arange(7), 8, 10000.0, dtype=torch.float64)
    for inter in (False, True):
        y = ref.rope_apply(x, cos, sin, inter)
        back = ref.rope_apply(y, cos, sin, inter, inverse=True)
        torch.testing.assert_close(back, x, atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4, rtol=1e-4)


def test_attention_varlen_matches_sdpa():
    torch.manual_seed(2)
    q = torch.randn(12, 4, 8)
    k = torch.randn(12, 2, 8)
    v = torch.randn(12, 2, 8)
    cu = torch.tensor([0, 5, 12], dtype=torch.int32)
    out = ref.attention_varlen(q, k, v, cu, cu, causal=True)
    for s, e in ((0, 5), (5, 12)):
        exp = torch.nn.functional.scaled_dot_product_attention(q[s:e].transpose(0, 1)[None], k[s:e].transpose(0, 1)[None], v[s:e].transpose(0, 1)[None], is_causal=True, enable_gqa=True)[0].transpose(0, 1)
        torch.testing.assert_close(out[s:e], exp, atol=1e-5, rtol=1e-5)


def test_sharded_cross_entropy_single_rank_matches_torch():
    from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy, sharded_cross_entropy_with_z_loss

    torch.manual_seed(3)
    logits = torch.randn(10, 50, dtype=torch.float32, requires_grad=True)
    tgt = torch.randint(0, 50, (10,))
    loss = sharded_cross_entropy(logits, tgt, group=None)
    exp = torch.nn.functional.cross_entropy(logits.detach().clone().requires_grad_(True), tgt, reduction="none")
    torch.testing.assert_close(loss, exp, atol=1e-5, rtol=1e-5)
    loss.mean().backward()
    l2 = logits.detach().clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(l2, tgt).backward()
    torch.testing.assert_close(logits.grad, l2.grad, atol=1e-6, rtol=1e-5)
    # z-loss term and its gradient
    l3 = logits.detach().clone().requires_grad_(True)
    ce, z = sharded_cross_entropy_with_z_loss(l3, tgt, group=None, z_loss_coef=1e-2)
    (ce + z).mean().backward()
    l4 = logits.detach().clone().requires_grad_(True)
    lz = torch.logsumexp(l4, -1)
    (torch.nn.functional.cross_entropy(l4, tgt, reduction="none") + 1e-2 * lz**2).mean().backward()
    torch.testing.assert_close(l3.grad, l4.grad, atol=1e-6, rtol=1e-4)


def test_adamw_reference_matches_torch():
    p = torch.randn(20)
    g = torch.randn(20)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(20), torch.zeros(20)
    for step in range(1, 4):
        ref_p.grad = g.clone()
        opt.step()
        ref.adamw_step(p, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    torch.testing.assert_close(p, ref_p.detach(), atol=1e-6, rtol=1e-5)


def test_rms_norm_return_input_fuses_the_skip_gradient():
    """``rms_norm(x, return_input=True)`` hands ``x`` back as a second output; gradients that reach it are summed into dx by the
    norm's own backward.  Compare with plain autograd where ``x`` feeds both the norm and the skip connection."""
    torch.manual_seed(0)
    x0 = torch.randn(6, 32, dtype=torch.float64)
    w0 = torch.randn(32, dtype=torch.float64)
    x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    y, skip = ops.rms_norm(x, w, 1e-5, return_input=True)
    ((y * y).sum() + (skip * 3).sum() + (y.sum(-1, keepdim=True) * skip).sum()).backward()
    xr, wr = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    ((yr * yr).sum() + (xr * 3).sum() + (yr.sum(-1, keepdim=True) * xr).sum()).backward()
    torch.testing.assert_close(x.grad, xr.grad, atol=1e-4, rtol=1e-4)  # the oracle keeps fp32 statistics
    torch.testing.assert_close(w.grad, wr.grad, atol=1e-4, rtol=1e-4)
    # the skip output alone
    x2 = x0.clone().requires_grad_(True)
    _, skip2 = ops.rms_norm(x2, w0, 1e-5, return_input=True)
    skip2.sum().backward()
    torch.testing.assert_close(x2.grad, torch.ones_like(x2))
