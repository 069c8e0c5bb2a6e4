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


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [([128], 1, 1, True), ([256], 2, 1, True), ([200, 56, 333], 4, 2, True), ([512, 100], 2, 2, False), ([1024], 8, 2, True)])
def test_flash_fwd_matches_oracle(lens, Hq, Hkv, causal):
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


def test_flash_fwd_sliding_window():
    from nanotron_b200.ops import native, native_attn

    native.lib()
    q, k, v = _qkv(700, 2, 1, seed=3)
    cu = torch.tensor([0, 300, 700], dtype=torch.int32, device=DEV)
    out, _ = native_attn.flash_attn_fwd(q, k, v, cu, cu, 400, 400, True, 0.088, 160)
    exp = ref.attention_varlen(q, k, v, cu, cu, causal=True, softmax_scale=0.088, window=160)
    torch.testing.assert_close(out.float(), exp.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [([128], 1, 1, True), ([256], 2, 1, True), ([200, 56, 333], 4, 2, True), ([384, 100], 2, 2, False), ([1024], 8, 2, True)])
def test_flash_bwd_matches_oracle(lens, Hq, Hkv, causal):
    from nanotron_b200 import ops
    from nanotron_b200.ops import native, native_gemm

    native.lib()
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
