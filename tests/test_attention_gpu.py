"""In-tree flash attention against the fp32 PyTorch oracle: causal / full, GQA, packed variable-length sequences,
strided q/k/v views of a fused qkv buffer."""
import math

import pytest
import torch

from nanotron_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _qkv(T, Hq, Hkv, seed=0):
    torch.manual_seed(seed)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device=DEV, dtype=torch.bfloat16)
    q = qkv[:, : Hq * 128].view(T, Hq, 128)
    k = qkv[:, Hq * 128 : (Hq + Hkv) * 128].view(T, Hkv, 128)
    v = qkv[:, (Hq + Hkv) * 128 :].view(T, Hkv, 128)
    return q, k, v


@pytest.fixture(params=["two_tile", "one_tile"])
def fwd_variant(request):
    """Both forward kernels: two query tiles per CTA with P in tensor memory (default), one query tile per CTA."""
    from nanotron_b200.ops import native_attn

    native_attn.set_forward_variant(request.param)
    yield request.param
    native_attn.set_forward_variant("two_tile")


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [([128], 1, 1, True), ([256], 2, 1, True), ([200, 56, 333], 4, 2, True), ([512, 100], 2, 2, False), ([1024], 8, 2, True), ([1300, 257, 640], 2, 1, True)])
def test_flash_fwd_matches_oracle(lens, Hq, Hkv, causal, fwd_variant):
    from nanotron_b200.ops import native, native_attn, native_gemm

    native.lib()
    T = sum(lens)
    q, k, v = _qkv(T, Hq, Hkv)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(128)
    out, lse = native_attn.flash_attn_fwd(q, k, v, cu, cu, max(lens), max(lens), causal, scale, None)
    native_gemm.check_status(DEV)
    exp, exp_lse = ref.attention_varlen(q, k, v, cu, cu, causal=causal, softmax_scale=scale, return_lse=True)
    torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse, exp_lse, atol=2e-2, rtol=1e-3)


def test_flash_fwd_large_logits_move_the_running_maximum(fwd_variant):
    """Scores whose row maximum keeps growing along the keys (by far more than the lazy-rescale threshold of the two-tile kernel)."""
    from nanotron_b200.ops import native, native_attn, native_gemm

    native.lib()
    T, Hq, Hkv = 1024, 2, 1
    q, k, v = _qkv(T, Hq, Hkv, seed=11)
    ramp = torch.linspace(0.2, 3.0, T, device=DEV).view(T, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)  # later keys give larger scores
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    scale = 0.5
    for causal in (True, False):
        out, lse = native_attn.flash_attn_fwd(q, k, v, cu, cu, T, T, causal, scale, None)
        native_gemm.check_status(DEV)
        exp, exp_lse = ref.attention_varlen(q, k, v, cu, cu, causal=causal, softmax_scale=scale, return_lse=True)
        torch.testing.assert_close(out.float(), exp.float(), atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(lse, exp_lse, atol=2e-2, rtol=1e-3)


def test_flash_fwd_sliding_window(fwd_variant):
    from nanotron_b200.ops import native, native_attn

    native.lib()
    q, k, v = _qkv(700, 2, 1, seed=3)
    cu = torch.tensor([0, 300, 700], dtype=torch.int32, device=DEV)
    out, _ = native_attn.flash_attn_fwd(q, k, v, cu, cu, 400, 400, True, 0.088, 160)
    exp = ref.attention_varlen(q, k, v, cu, cu, causal=True, softmax_scale=0.088, window=160)
    torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("split", ["off", "on"])
@pytest.mark.parametrize("lens,Hq,Hkv,causal", [([128], 1, 1, True), ([256], 2, 1, True), ([200, 56, 333], 4, 2, True), ([384, 100], 2, 2, False), ([1024], 8, 2, True)])
def test_flash_bwd_matches_oracle(lens, Hq, Hkv, causal, split, monkeypatch):
    """``split``: one backward CTA per kv head (dK / dV in tensor memory to the end) or per query head (fp32 accumulation across the
    query heads of a group, what small launches select by themselves)."""
    from nanotron_b200 import ops
    from nanotron_b200.ops import native, native_attn, native_gemm

    native.lib()
    monkeypatch.setitem(native_attn.BWD_SPLIT, "mode", split)
    T = sum(lens)
    q, k, v = _qkv(T, Hq, Hkv, seed=5)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(128)
    qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    ops.set_attention("native")
    try:
        out = ops.flash_attn_varlen(qg, kg, vg, cu, cu, max(lens), max(lens), causal=causal, softmax_scale=scale)
        g = torch.randn_like(out)
        out.backward(g)
    finally:
        ops.set_attention("auto")
    native_gemm.check_status(DEV)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    exp = ref.attention_varlen(qf, kf, vf, cu, cu, causal=causal, softmax_scale=scale)
    exp.backward(g.float())
    for name, a, b in (("dq", qg.grad, qf.grad), ("dk", kg.grad, kf.grad), ("dv", vg.grad, vf.grad)):
        err = (a.float() - b).abs().max().item()
        ref_mag = b.abs().max().item()
        assert err < 3e-2 * max(ref_mag, 1.0), f"{name}: max err {err} vs magnitude {ref_mag}"


def test_fused_qkv_rope_attention_matches_composition():
    """RoPE + attention on the fused projection output with one gradient buffer == rotate q / k, attend, differentiate (fp32)."""
    from nanotron_b200 import ops

    lens, Hq, Hkv, D = [200, 312], 4, 2, 128
    T = sum(lens)
    cu = torch.tensor([0, 200, 512], dtype=torch.int32, device=DEV)
    positions = torch.cat([torch.arange(n, device=DEV) for n in lens])
    cos, sin = ref.rope_cos_sin(torch.arange(512, device=DEV), D, 10000.0)
    torch.manual_seed(3)
    qkv0 = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
    g = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    # oracle in fp32
    x = qkv0.float().requires_grad_(True)
    q = x[:, : Hq * D].view(T, Hq, D)
    k = x[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = x[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    c, s_ = cos[positions], sin[positions]
    qr, kr = ref.rope_apply(q, c, s_, False), ref.rope_apply(k, c, s_, False)
    exp = ref.attention_varlen(qr, kr, v, cu, cu, causal=True, softmax_scale=1 / math.sqrt(D))
    exp.backward(g.float())
    # fused op (it rotates its input in place: give it a copy)
    ops.set_attention("native")
    try:
        y = qkv0.clone().requires_grad_(True)
        buf = y * 1  # non-leaf, as the projection output is
        assert ops.fused_qkv_attention_supported(buf, Hq, Hkv, D, None)
        out = ops.fused_qkv_attention(buf, cos, sin, positions, Hq, Hkv, D, cu, max(lens))
        out.backward(g)
    finally:
        ops.set_attention("auto")
    torch.testing.assert_close(out.float(), exp.detach(), atol=3e-2, rtol=3e-2)
    err = (y.grad.float() - x.grad).abs().max() / x.grad.abs().max()
    assert err < 3e-2, float(err)


def test_fused_qkv_library_attention_matches_composition():
    """The fusion around the library attention (in-place RoPE, one qkv gradient buffer) == rotate, attend, differentiate in fp32."""
    from nanotron_b200 import ops

    B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
    T = B * S
    cu = torch.tensor([0, S, 2 * S], dtype=torch.int32, device=DEV)
    positions = torch.arange(S, device=DEV).repeat(B)
    cos, sin = ref.rope_cos_sin(torch.arange(S, device=DEV), D, 10000.0)
    torch.manual_seed(5)
    qkv0 = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
    g = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    x = qkv0.float().requires_grad_(True)
    q = x[:, : Hq * D].view(T, Hq, D)
    k = x[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = x[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    c, s_ = cos[positions], sin[positions]
    exp = ref.attention_varlen(ref.rope_apply(q, c, s_, False), ref.rope_apply(k, c, s_, False), v, cu, cu, causal=True, softmax_scale=1 / math.sqrt(D))
    exp.backward(g.float())
    y = qkv0.clone().requires_grad_(True)
    buf = y * 1
    assert ops.fused_qkv_library_attention_supported(buf, D, None, None)
    out = ops.fused_qkv_library_attention(buf, cos, sin, positions, Hq, Hkv, D, B, S)
    out.backward(g)
    torch.testing.assert_close(out.float(), exp.detach(), atol=3e-2, rtol=3e-2)
    err = (y.grad.float() - x.grad).abs().max() / x.grad.abs().max()
    assert err < 3e-2, float(err)
    # no-grad call (generation / evaluation)
    with torch.no_grad():
        out2 = ops.fused_qkv_library_attention(qkv0.clone(), cos, sin, positions, Hq, Hkv, D, B, S)
    torch.testing.assert_close(out2, out.detach())


@pytest.mark.parametrize("mode", ["auto", "sdpa"])
@pytest.mark.parametrize("lq,lk,window", [(64, 192, None), (128, 384, None), (256, 256, 100), (128, 512, 200)])
def test_default_path_causal_mask_is_bottom_right_aligned(mode, lq, lk, window):
    """Fewer queries than keys (what context parallelism produces): query i of a row sees keys <= i + lk - lq, on the default
    path (in-tree kernel) and on the library path alike; both must match the fp32 oracle, forward and gradients."""
    from nanotron_b200 import ops

    B, Hq, Hkv, D = 2, 4, 2, 128
    torch.manual_seed(lq + lk)
    q = torch.randn(B * lq, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B * lk, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B * lk, Hkv, D, device=DEV, dtype=torch.bfloat16)
    cu_q = torch.arange(0, (B + 1) * lq, lq, dtype=torch.int32, device=DEV)
    cu_k = torch.arange(0, (B + 1) * lk, lk, dtype=torch.int32, device=DEV)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    ops.set_attention(mode)
    try:
        out = ops.flash_attn_varlen(qg, kg, vg, cu_q, cu_k, lq, lk, causal=True, window=window)
        g = torch.randn_like(out)
        out.backward(g)
    finally:
        ops.set_attention("auto")
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    exp = ref.attention_varlen(qf, kf, vf, cu_q, cu_k, causal=True, window=window)
    exp.backward(g.float())
    torch.testing.assert_close(out.float(), exp.detach(), atol=2e-2, rtol=2e-2)
    for name, a, b in (("dq", qg.grad, qf.grad), ("dk", kg.grad, kf.grad), ("dv", vg.grad, vf.grad)):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * max(b.abs().max().item(), 1.0), f"{name}: {err}"


@pytest.mark.parametrize("mode", ["auto", "sdpa"])
def test_default_path_ragged_documents_and_toy_head_dim(mode):
    """Packed documents of unequal length: head dim 128 runs the in-tree kernel, head dim 64 (outside its contract) the library
    kernel per document -- neither may fall back to anything that differs from the oracle."""
    from nanotron_b200 import ops

    lens = [100, 37, 300, 75]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ops.set_attention(mode)
    try:
        for D in (128, 64):
            torch.manual_seed(D)
            q = torch.randn(T, 4, D, device=DEV, dtype=torch.bfloat16)
            k = torch.randn(T, 2, D, device=DEV, dtype=torch.bfloat16)
            v = torch.randn(T, 2, D, device=DEV, dtype=torch.bfloat16)
            import warnings

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                out = ops.flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=True, window=64)
            exp = ref.attention_varlen(q, k, v, cu, cu, causal=True, window=64)
            torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)
    finally:
        ops.set_attention("auto")


def test_registry_backends_agree_on_cuda():
    """"flash_attention_2", "sdpa" and "flex_attention" (document + window mask) give the oracle's result on CUDA tensors."""
    from nanotron_b200.nn.attention import ALL_ATTENTION_FUNCTIONS

    lens = [256, 128, 200]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _qkv(T, 4, 2, seed=21)
    exp = ref.attention_varlen(q, k, v, cu, cu, causal=True, window=96)
    for name, kw in (("flash_attention_2", {}), ("sdpa", {}), ("flex_attention", {"flex_attention_mask": "sliding_window_document"})):
        out = ALL_ATTENTION_FUNCTIONS[name](q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens), causal=True, sliding_window=96, **kw)
        torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)
    # the window-only mask ignores the document boundaries
    one = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    exp = ref.attention_varlen(q, k, v, one, one, causal=True, window=96)
    out = ALL_ATTENTION_FUNCTIONS["flex_attention"](q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens), causal=True, sliding_window=96, flex_attention_mask="sliding_window")
    torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)
