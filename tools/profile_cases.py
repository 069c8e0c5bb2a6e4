"""Small, self-ending workloads for profiler captures: each in-tree kernel runs twice (one warm-up, one measured) on inputs
larger than the L2 cache but well under a gigabyte or two in total, so a counter capture replays quickly.

    python tools/profile_cases.py [gemm|norm|elementwise|attention|moe|optim|all]
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import math

import torch


def _twice(fn):
    fn()
    fn()
    torch.cuda.synchronize()


def case_gemm():
    from nanotron_b200.ops import native_gemm as g

    M, N, K = 8192, 6144, 4096  # x 64 MiB, w 48 MiB, y 96 MiB
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    for variant in ("single", "pair"):
        g.set_variant(variant)
        _twice(lambda: g.gemm_nt(x, w))
        _twice(lambda: g.gemm_nn(dy, w))
        _twice(lambda: g.gemm_tn_accum_fp32(dy, x, acc))
    g.check_status("cuda")


def case_norm():
    from nanotron_b200.ops import native

    T, H = 16384, 4096  # 128 MiB per tensor
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y, pre, rstd = native.rmsnorm_fwd(x, r, w, 1e-5)
    _twice(lambda: native.rmsnorm_fwd(x, r, w, 1e-5))
    _twice(lambda: native.rmsnorm_bwd(y, pre, w, rstd, r))


def case_elementwise():
    from nanotron_b200.ops import native
    from nanotron_b200.ops import reference as ref

    T, I, V = 8192, 14336, 128256
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    _twice(lambda: native.swiglu_fwd(gu))
    _twice(lambda: native.swiglu_bwd(gu, do))
    Tq = 32768
    qkv = torch.randn(Tq, 6144, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, :4096].view(Tq, 32, 128)
    pos = torch.arange(Tq, device="cuda") % 4096
    cos, sin = ref.rope_cos_sin(torch.arange(4096, device="cuda"), 128, 500000.0)
    _twice(lambda: native.rope(q, cos, sin, False, False, True, positions=pos))
    logits = torch.randn(2048, V, device="cuda", dtype=torch.bfloat16)
    tgt = torch.randint(0, V, (2048,), device="cuda")
    m, s, t = native.ce_partials(logits, tgt, 0)
    logz = m + torch.log(s)
    gl = torch.ones(2048, device="cuda")
    _twice(lambda: native.ce_partials(logits, tgt, 0))
    _twice(lambda: native.ce_backward(logits, tgt, logz, gl, None, 0, inplace=True))


def case_attention():
    from nanotron_b200.ops import native_attn, native_gemm

    B, S, Hq, Hkv = 2, 4096, 32, 8
    T = B * S
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : Hq * 128].view(T, Hq, 128)
    k = qkv[:, Hq * 128 : (Hq + Hkv) * 128].view(T, Hkv, 128)
    v = qkv[:, (Hq + Hkv) * 128 :].view(T, Hkv, 128)
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(128)
    out, lse = native_attn.flash_attn_fwd(q, k, v, cu, cu, S, S, True, scale, None)
    dout = torch.randn_like(out)
    _twice(lambda: native_attn.flash_attn_fwd(q, k, v, cu, cu, S, S, True, scale, None))
    _twice(lambda: native_attn.flash_attn_bwd(dout, q, k, v, out, lse, cu, cu, S, S, True, scale, None))
    native_gemm.check_status("cuda")


def case_moe():
    from nanotron_b200.ops import moe_fused, native

    T, E, k, h, inter = 8192, 64, 4, 2048, 1408
    x = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    wr = torch.randn(E, h, device="cuda", dtype=torch.float32) * 0.02
    top_p, top_i, probs, counts = native.moe_router_fwd(x, wr, k)
    _twice(lambda: native.moe_router_fwd(x, wr, k))
    ctx = moe_fused.get_context(None, h, T, k, E)
    plan = ctx.make_plan(counts, top_i)
    _twice(lambda: ctx.make_plan(counts, top_i))
    _twice(lambda: ctx.dispatch(x, top_i, plan, None, zero_pad=True))
    w1 = (torch.randn(E, h, 2 * inter, device="cuda") * 0.02).to(torch.bfloat16)
    xp = ctx.recv.tensor.view(ctx.cap_rows, h).clone()
    _twice(lambda: ctx.grouped(xp, w1, True, plan))
    ctx.ybuf.tensor.copy_(ctx.recv.tensor)
    _twice(lambda: ctx.combine(top_i, plan, top_p, T, False))
    ctx.check()


def case_optim():
    from nanotron_b200.ops import native

    n = 64 * 1024 * 1024
    p, g_, m_, v_ = (torch.zeros(n, device="cuda") for _ in range(4))
    p16 = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    seg_end = torch.tensor([n], dtype=torch.int64, device="cuda")
    seg_lr = torch.tensor([1e-3], device="cuda")
    seg_wd = torch.tensor([0.01], device="cuda")
    _twice(lambda: native.adamw_flat(p, g_, m_, v_, p16, seg_end, seg_lr, seg_wd, 0.9, 0.95, 1e-8, 1.0))
    _twice(lambda: native.sumsq(g_))


CASES = {"gemm": case_gemm, "norm": case_norm, "elementwise": case_elementwise, "attention": case_attention, "moe": case_moe, "optim": case_optim}

if __name__ == "__main__":
    from nanotron_b200.ops import native

    native.lib()
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    for name, fn in CASES.items():
        if what in ("all", name):
            fn()
            torch.cuda.empty_cache()
            print(f"{name}: done", flush=True)
