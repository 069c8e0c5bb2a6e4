"""Numerics of every in-tree CUDA kernel against the PyTorch fp32 oracle (small shapes incl. ragged edges)."""
import math

import pytest
import torch

from nanotron_b200 import ops
from nanotron_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, what=""):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol, msg=lambda m: f"{what}: {m}")


@pytest.mark.parametrize("rows,cols", [(7, 64), (33, 1024), (128, 4096), (5, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, cols, dtype, with_res):
    from nanotron_b200.ops import native

    torch.manual_seed(0)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype)
    r = torch.randn(rows, cols, device=DEV, dtype=dtype) if with_res else None
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(dtype)
    y, pre, rstd = native.rmsnorm_fwd(x, r, w, 1e-5)
    y0, pre0, rstd0 = ref.rms_norm_fwd(x, w, 1e-5, r)
    tol = dict(atol=2e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    _close(y, y0, what="y", **tol)
    _close(pre, pre0, what="pre", **tol)
    _close(rstd, rstd0, atol=1e-4, rtol=1e-4, what="rstd")
    dy = torch.randn(rows, cols, device=DEV, dtype=dtype)
    dres = torch.randn(rows, cols, device=DEV, dtype=dtype) if with_res else None
    dx, dw = native.rmsnorm_bwd(dy, pre, w, rstd, dres)
    dx0, dw0 = ref.rms_norm_bwd(dy, pre0, w, rstd0, dres)
    _close(dx, dx0, what="dx", **tol)
    _close(dw, dw0, atol=5e-2 if dtype == torch.bfloat16 else 1e-3, rtol=2e-2, what="dw")


@pytest.mark.parametrize("rows,cols", [(9, 128), (64, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layernorm(rows, cols, dtype):
    from nanotron_b200.ops import native

    torch.manual_seed(1)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype) + 0.5
    r = torch.randn(rows, cols, device=DEV, dtype=dtype)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(dtype)
    b = (0.1 * torch.randn(cols, device=DEV)).to(dtype)
    y, pre, mean, rstd = native.layernorm_fwd(x, r, w, b, 1e-5)
    y0, pre0, mean0, rstd0 = ref.layer_norm_fwd(x, w, b, 1e-5, r)
    tol = dict(atol=3e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    _close(y, y0, what="y", **tol)
    dy = torch.randn(rows, cols, device=DEV, dtype=dtype)
    dx, dw, db = native.layernorm_bwd(dy, pre, w, mean, rstd, None, True)
    dx0, dw0, db0 = ref.layer_norm_bwd(dy, pre0, w, mean0, rstd0, None, True)
    _close(dx, dx0, what="dx", **tol)
    _close(dw, dw0, atol=5e-2 if dtype == torch.bfloat16 else 1e-3, rtol=2e-2, what="dw")
    _close(db, db0, atol=5e-2 if dtype == torch.bfloat16 else 1e-3, rtol=2e-2, what="db")


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_strided_views(interleaved, dtype):
    torch.manual_seed(2)
    T, Hq, Hkv, D = 37, 4, 2, 64
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, dtype=dtype)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    pos = torch.randint(0, 100, (T,), device=DEV)
    cos_t, sin_t = ref.rope_cos_sin(torch.arange(128, device=DEV), D, 10000.0)
    cos, sin = cos_t[pos], sin_t[pos]
    for x in (q, k):
        out = ops.apply_rotary(x, cos_t.contiguous(), sin_t.contiguous(), interleaved, False, positions=pos)
        exp = ref.rope_apply(x, cos, sin, interleaved)
        _close(out, exp, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2, what="rope fwd")
    # backward is the inverse rotation
    xg = q.clone().requires_grad_(True)
    out = ops.apply_rotary(xg, cos_t.contiguous(), sin_t.contiguous(), interleaved, False, positions=pos)
    g = torch.randn_like(out)
    out.backward(g)
    exp = ref.rope_apply(g, cos, sin, interleaved, inverse=True)
    _close(xg.grad, exp, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2, what="rope bwd")


@pytest.mark.parametrize("rows,inter", [(5, 64), (130, 1408), (64, 14336)])
def test_swiglu(rows, inter):
    torch.manual_seed(3)
    gu = torch.randn(rows, 2 * inter, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = ops.swiglu(gu)
    _close(out, ref.swiglu_fwd(gu), atol=2e-2, rtol=2e-2, what="swiglu fwd")
    d = torch.randn_like(out)
    out.backward(d)
    _close(gu.grad, ref.swiglu_bwd(gu, d), atol=3e-2, rtol=3e-2, what="swiglu bwd")


@pytest.mark.parametrize("rows,vocab,start", [(4, 256, 0), (19, 32064, 32064), (8, 128256, 0)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_pieces(rows, vocab, start, dtype):
    from nanotron_b200.ops import native

    torch.manual_seed(4)
    logits = (3 * torch.randn(rows, vocab, device=DEV)).to(dtype)
    tgt = torch.randint(0, 2 * vocab, (rows,), device=DEV)
    m, s, t = native.ce_partials(logits, tgt, start)
    m0, s0, t0 = ref.ce_partials(logits, tgt, start)
    _close(m, m0, atol=1e-6, rtol=0, what="max")
    _close(s, s0, atol=1e-2, rtol=1e-3, what="sumexp")
    _close(t, t0, atol=1e-6, rtol=0, what="target logit")
    logz = m0 + torch.log(s0)
    g = torch.rand(rows, device=DEV)
    gz = 0.01 * torch.rand(rows, device=DEV)
    exp = ref.ce_backward(logits, tgt, logz, g, gz, start)
    got = native.ce_backward(logits.clone(), tgt, logz, g, gz, start, inplace=True)
    _close(got, exp, atol=1e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2, what="dlogits")


def test_sharded_cross_entropy_matches_torch():
    from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy

    torch.manual_seed(5)
    logits = torch.randn(64, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    tgt = torch.randint(0, 1024, (64,), device=DEV)
    ref_logits = logits.detach().float().requires_grad_(True)
    loss = sharded_cross_entropy(logits, tgt, group=None).mean()
    exp = torch.nn.functional.cross_entropy(ref_logits, tgt)
    _close(loss, exp, atol=1e-3, rtol=1e-3, what="loss")
    loss.backward()
    exp.backward()
    _close(logits.grad, ref_logits.grad, atol=1e-4, rtol=5e-2, what="grad")


def test_adamw_flat_matches_torch():
    from nanotron_b200.optim.fused_adamw import FusedAdamW

    torch.manual_seed(6)
    sizes = [(128, 64), (384,), (256, 8)]
    total = sum(math.prod(s) for s in sizes)
    master = torch.randn(total, device=DEV)
    grads = torch.randn(total, device=DEV)
    half = torch.zeros(total, device=DEV, dtype=torch.bfloat16)
    params, refs, off = [], [], 0
    opt_groups = []
    for i, s in enumerate(sizes):
        n = math.prod(s)
        p = torch.nn.Parameter(master[off : off + n].view(s))
        p.grad = grads[off : off + n].view(s)
        params.append(p)
        refs.append(torch.nn.Parameter(p.detach().clone()))
        refs[-1].grad = p.grad.clone()
        off += n
    wds = [0.1, 0.0, 0.1]
    opt = FusedAdamW([{"params": [p], "weight_decay": wd} for p, wd in zip(params, wds)], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    off = 0
    for p in params:
        opt.set_half_target(p, half[off : off + p.numel()])
        off += p.numel()
    scale = torch.tensor(0.5, device=DEV)
    opt.grad_scale = scale
    tref = torch.optim.AdamW([{"params": [p], "weight_decay": wd} for p, wd in zip(refs, wds)], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(3):
        for r in refs:
            r.grad = r.grad * 0 + grads[: 0].new_tensor(0)  # placeholder overwritten below
        off = 0
        for r in refs:
            r.grad = grads[off : off + r.numel()].view(r.shape) * 0.5
            off += r.numel()
        opt.step()
        tref.step()
    assert opt._flat is not None, "expected the single-launch flat path"
    for p, r in zip(params, refs):
        _close(p, r, atol=1e-5, rtol=1e-5, what="param")
    _close(half, master, atol=1e-2, rtol=1e-2, what="bf16 copy")


def test_sumsq():
    from nanotron_b200.ops import native

    x = torch.randn(1_000_003, device=DEV)
    xa = torch.empty(1_000_004, device=DEV)[:1_000_003].copy_(x)
    got = native.sumsq(xa)
    _close(got.squeeze(), x.double().pow(2).sum().float(), atol=0, rtol=1e-4, what="sumsq")


@pytest.mark.parametrize("T,h,E,k", [(50, 256, 16, 2), (1000, 2048, 64, 4), (33, 512, 128, 8)])
def test_moe_router_kernel(T, h, E, k):
    from nanotron_b200.ops import native

    torch.manual_seed(7)
    x = torch.randn(T, h, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(E, h, device=DEV) * 0.05
    top_p, top_i, probs, counts = native.moe_router_fwd(x, w, k)
    exp_probs = torch.softmax(x.float() @ w.t(), dim=-1)
    _close(probs, exp_probs, atol=1e-5, rtol=1e-4, what="probs")
    exp_p, exp_i = torch.topk(exp_probs, k, dim=-1)
    _close(top_p, exp_p, atol=1e-5, rtol=1e-4, what="top probs")
    # ties aside, the same experts are chosen
    assert (top_i.long() == exp_i).float().mean() > 0.999
    assert int(counts.sum()) == T * k
    assert torch.equal(counts.long(), torch.bincount(top_i.reshape(-1).long(), minlength=E))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_masked_embedding_forward_and_fp32_accumulating_backward(dtype):
    from nanotron_b200 import ops

    V, h, n = 1000, 256, 777
    min_id, max_id = 250, 500
    torch.manual_seed(0)
    w = torch.randn(max_id - min_id, h, device="cuda", dtype=dtype, requires_grad=True)
    ids = torch.randint(0, V, (7, 111), device="cuda")
    out = ops.masked_embedding(ids, w, min_id, max_id)
    mask = (ids < min_id) | (ids >= max_id)
    exp = torch.nn.functional.embedding((ids - min_id).masked_fill(mask, 0), w.detach()).masked_fill(mask.unsqueeze(-1), 0.0)
    assert torch.equal(out, exp)
    g = torch.randn_like(out)
    # plain gradient
    out.backward(g)
    exp_dw = torch.zeros(max_id - min_id, h, device="cuda", dtype=torch.float32)
    exp_dw.index_add_(0, (ids - min_id).masked_fill(mask, 0).reshape(-1), (g.float() * (~mask).unsqueeze(-1)).reshape(-1, h))
    torch.testing.assert_close(w.grad.float(), exp_dw, atol=3e-2 if dtype == torch.bfloat16 else 1e-4, rtol=2e-2)
    # accumulation into an fp32 main-gradient buffer
    w.grad = None
    w.main_grad = torch.full((max_id - min_id, h), 0.25, device="cuda", dtype=torch.float32)
    ops.masked_embedding(ids, w, min_id, max_id).backward(g)
    assert w.grad is None
    torch.testing.assert_close(w.main_grad, exp_dw + 0.25, atol=1e-4, rtol=1e-4)


def test_device_side_wait_gives_up_and_reports():
    """A wait on a flag that nothing sets must run out after its limit, set the status word and leave the context usable."""
    import ctypes
    import time

    from nanotron_b200.ops import native

    L = native.lib()
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.ntb_symm_wait.restype = ctypes.c_int
    L.ntb_symm_wait.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
    torch.cuda.synchronize()
    t0 = time.time()
    rc = L.ntb_symm_wait(flags.data_ptr(), 2, 1, 50_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)  # 50 ms
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(status.item()) == 3  # NTB_ERR_TIMEOUT
    # the same wait succeeds at once when the flags carry the epoch, and ordinary kernels still run
    flags.fill_(1)
    status.zero_()
    assert L.ntb_symm_wait(flags.data_ptr(), 2, 1, 50_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def test_rms_norm_return_input_sums_the_skip_gradient_in_the_kernel():
    """`ops.rms_norm(x, return_input=True)` on the native path: the gradient reaching the second output (the skip connection) is
    added by the norm's backward kernel.  Compared with fp32 autograd where `x` feeds the norm and the skip separately."""
    torch.manual_seed(4)
    T, H = 384, 1024
    x0 = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w0 = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    gy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    gs = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    y, skip = ops.rms_norm(x, w, 1e-5, return_input=True)
    torch.autograd.backward([y, skip], [gy, gs])
    xr, wr = x0.float().requires_grad_(True), w0.float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    torch.autograd.backward([yr, xr * 1.0], [gy.float(), gs.float()])
    torch.testing.assert_close(y.float(), yr.detach(), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=5e-2, rtol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.5, rtol=5e-2)


def test_rotary_on_a_toy_head_dim_takes_the_composition():
    """Head dim 4 (the toy example config) is outside the RoPE kernel's contract (multiples of 16, 16-byte rows): `apply_rotary`
    must still work on the GPU, forward and backward, through the PyTorch composition."""
    torch.manual_seed(1)
    T, H, D = 32, 4, 4
    qkv = torch.randn(T, 3 * H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q = qkv[:, : H * D].view(T, H, D)
    pos = torch.arange(T, device="cuda")
    cos, sin = ref.rope_cos_sin(torch.arange(64, device="cuda"), D, 10000.0)
    out = ops.apply_rotary(q, cos, sin, False, False, positions=pos)
    exp = ref.rope_apply(q.detach().float(), cos[pos], sin[pos], False)
    torch.testing.assert_close(out.float(), exp, atol=2e-2, rtol=2e-2)
    out.float().sum().backward()
    assert qkv.grad is not None and torch.isfinite(qkv.grad).all()
