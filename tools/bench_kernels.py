"""Micro-benchmarks of the in-tree kernels against their roofline (run on a B200).

    python tools/bench_kernels.py gemm            # tcgen05 GEMM vs the library GEMM on Llama-3-8B shapes
    python tools/bench_kernels.py gemm-split      # tensor-parallel per-rank shapes: last round split along K vs whole tiles
    python tools/bench_kernels.py elementwise     # HBM-bound kernels vs measured copy bandwidth
    python tools/bench_kernels.py attention

Timing: CUDA events, 3 warm-up + 10 timed launches; operands are rotated through several buffers so that consecutive
launches do not find their inputs in L2 (total footprint > 126 MB).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import json

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "_fallback": True}


def time_fn(fn, n_warm=3, n_iter=10) -> float:
    """Milliseconds per call."""
    for _ in range(n_warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n_iter):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / n_iter


def bench_gemm(small: bool = False):
    from nanotron_b200.ops import native, native_gemm as g

    native.lib()
    peak = _peaks()["bf16_tflops"]
    shapes = [("qkv", 4096, 6144, 4096), ("o", 4096, 4096, 4096), ("gate_up", 4096, 28672, 4096), ("down", 4096, 4096, 14336), ("lm_head", 4096, 128256, 4096)]
    if small:
        shapes = [("qkv", 4096, 6144, 4096)]
    for name, M, N, K in shapes:
        nbuf = max(2, int(300e6 // ((M * K + N * K) * 2)) + 1)
        xs = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
        dys = [torch.randn(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        i = [0]

        def nxt():
            i[0] = (i[0] + 1) % nbuf
            return i[0]

        flops = 2.0 * M * N * K
        rows = {}
        rows["fwd  tcgen05"] = time_fn(lambda: g.gemm_nt(xs[nxt()], ws[i[0]]))
        rows["fwd  library"] = time_fn(lambda: torch.nn.functional.linear(xs[nxt()], ws[i[0]]))
        rows["dgrad tcgen05"] = time_fn(lambda: g.gemm_nn(dys[nxt() % 2], ws[i[0]]))
        rows["dgrad library"] = time_fn(lambda: dys[nxt() % 2].matmul(ws[i[0]]))
        rows["wgrad tcgen05 (+= fp32)"] = time_fn(lambda: g.gemm_tn_accum_fp32(dys[nxt() % 2], xs[i[0]], acc))
        rows["wgrad library (bf16 out, then fp32 add)"] = time_fn(lambda: acc.add_(dys[nxt() % 2].t().matmul(xs[i[0]])))
        for k, ms in rows.items():
            tf = flops / ms / 1e9
            print(f"{name:8s} M={M} N={N} K={K}  {k:42s} {ms:8.3f} ms  {tf:7.1f} TFLOP/s  {tf / peak:5.2f} of measured peak", flush=True)
        g.check_status("cuda")
        del xs, ws, dys, acc
        torch.cuda.empty_cache()


def bench_gemm_split():
    """Per-rank Llama-3-8B shapes under tp 2 / tp 4, whose tile counts do not fill the last round of the 74 CTA pairs: the pair
    kernel with and without the split of that round along K, against the library GEMM."""
    from nanotron_b200.ops import native, native_gemm as g

    native.lib()
    peak = _peaks()["bf16_tflops"]
    shapes = [("qkv tp4", 4096, 1536, 4096), ("qkv tp2", 4096, 3072, 4096), ("o tp4 dgrad-like", 4096, 4096, 1024), ("gate_up tp4", 4096, 7168, 4096),
              ("gate_up tp2", 4096, 14336, 4096), ("down tp4", 4096, 4096, 3584), ("down tp2", 4096, 4096, 7168), ("qkv tp1", 4096, 6144, 4096)]
    for name, M, N, K in shapes:
        nbuf = max(2, int(300e6 // ((M * K + N * K) * 2)) + 1)
        xs = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
        dys = [torch.randn(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        i = [0]

        def nxt():
            i[0] = (i[0] + 1) % nbuf
            return i[0]

        flops = 2.0 * M * N * K
        rows = {}
        for label, on in (("split", True), ("whole tiles", False)):
            g.set_split(on)
            rows[f"fwd   pair kernel, {label}"] = time_fn(lambda: g.gemm_nt(xs[nxt()], ws[i[0]]))
            rows[f"dgrad pair kernel, {label}"] = time_fn(lambda: g.gemm_nn(dys[nxt() % 2], ws[i[0]]))
            rows[f"wgrad pair kernel (+= fp32), {label}"] = time_fn(lambda: g.gemm_tn_accum_fp32(dys[nxt() % 2], xs[i[0]], acc))
        g.set_split(False)
        rows["fwd   library"] = time_fn(lambda: torch.nn.functional.linear(xs[nxt()], ws[i[0]]))
        rows["dgrad library"] = time_fn(lambda: dys[nxt() % 2].matmul(ws[i[0]]))
        for k, ms in rows.items():
            tf = flops / ms / 1e9
            print(f"{name:18s} M={M} N={N} K={K}  {k:42s} {ms:8.3f} ms  {tf:7.1f} TFLOP/s  {tf / peak:5.2f} of measured peak", flush=True)
        g.check_status("cuda")
        del xs, ws, dys, acc
        torch.cuda.empty_cache()


def bench_elementwise():
    from nanotron_b200 import ops
    from nanotron_b200.ops import native

    native.lib()
    bw = _peaks()["hbm_gbs"]
    T, H, I, V = 8192, 4096, 14336, 128256
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y, pre, rstd = native.rmsnorm_fwd(x, r, w, 1e-5)
    cases = [
        ("rmsnorm fwd (+residual)", lambda: native.rmsnorm_fwd(x, r, w, 1e-5), 4 * T * H * 2),
        ("rmsnorm bwd (+residual)", lambda: native.rmsnorm_bwd(y, pre, w, rstd, r), 4 * T * H * 2),
    ]
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    cases += [
        ("swiglu fwd", lambda: native.swiglu_fwd(gu), 3 * T * I * 2),
        ("swiglu bwd", lambda: native.swiglu_bwd(gu, do), 5 * T * I * 2),
    ]
    qkv = torch.randn(T, 6144, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, :4096].view(T, 32, 128)
    from nanotron_b200.ops import reference as ref

    cos, sin = ref.rope_cos_sin(torch.arange(T, device="cuda"), 128, 500000.0)
    pos = torch.arange(T, device="cuda")
    cases.append(("rope (q, 32 heads, in place)", lambda: native.rope(q, cos, sin, False, False, True, positions=pos), 2 * T * 4096 * 2))
    logits = torch.randn(4096, V, device="cuda", dtype=torch.bfloat16)
    tgt = torch.randint(0, V, (4096,), device="cuda")
    m, s, t = native.ce_partials(logits, tgt, 0)
    logz = m + torch.log(s)
    gl = torch.ones(4096, device="cuda")
    cases += [
        ("cross-entropy partials", lambda: native.ce_partials(logits, tgt, 0), 4096 * V * 2),
        ("cross-entropy backward (in place)", lambda: native.ce_backward(logits, tgt, logz, gl, None, 0, inplace=True), 2 * 4096 * V * 2),
    ]
    n = 256 * 1024 * 1024
    p, g_, m_, v_ = (torch.zeros(n, device="cuda") for _ in range(4))
    p16 = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    seg_end = torch.tensor([n], dtype=torch.int64, device="cuda")
    seg_lr = torch.tensor([1e-3], device="cuda")
    seg_wd = torch.tensor([0.01], device="cuda")
    cases.append(("adamw flat (fp32 master + bf16 write-back)", lambda: native.adamw_flat(p, g_, m_, v_, p16, seg_end, seg_lr, seg_wd, 0.9, 0.95, 1e-8, 1.0), n * (4 * 4 + 3 * 4 + 2)))
    cases.append(("sum of squares (grad norm)", lambda: native.sumsq(g_), n * 4))
    for name, fn, nbytes in cases:
        ms = time_fn(fn)
        gbs = nbytes / ms / 1e6
        print(f"{name:46s} {ms:8.3f} ms  {gbs:8.1f} GB/s  {gbs / bw:5.2f} of measured copy bandwidth", flush=True)


def bench_moe():
    """Grouped expert GEMMs (tcgen05, device-side offsets) against the library grouped GEMM, and the dispatch / combine
    kernels against the copy-bandwidth roofline; 8192 tokens, top-4 of 64 experts, h = 2048, expert width 1408."""
    from nanotron_b200.ops import moe_fused, native

    native.lib()
    pk = _peaks()
    T, E, k, h, inter = 8192, 64, 4, 2048, 1408
    torch.manual_seed(0)
    probs = torch.softmax(torch.randn(T, E, device="cuda"), -1)
    top_p, top_i = torch.topk(probs, k, dim=-1)
    top_p, top_i = top_p.float().contiguous(), top_i.to(torch.int32).contiguous()
    counts = torch.bincount(top_i.reshape(-1), minlength=E).to(torch.int32)
    ctx = moe_fused.get_context(None, h, T, k, E)
    plan = ctx.make_plan(counts, top_i)
    x = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    w1 = (torch.randn(E, h, 2 * inter, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, inter, h, device="cuda") * 0.02).to(torch.bfloat16)
    cap = ctx.cap_rows
    rows = T * k
    ms = time_fn(lambda: ctx.make_plan(counts, top_i))
    print(f"plan + rank (T*k = {rows})                       {ms:8.3f} ms", flush=True)
    ms = time_fn(lambda: ctx.dispatch(x, top_i, plan, None, zero_pad=True))
    gbs = (T * h * 2 + rows * h * 2) / ms / 1e6
    print(f"dispatch (read T rows, write T*k rows)           {ms:8.3f} ms  {gbs:8.1f} GB/s  {gbs / pk['hbm_gbs']:5.2f} of measured copy bandwidth", flush=True)
    xp = ctx.recv.tensor.view(cap, h).clone()
    ctx.ybuf.tensor.copy_(ctx.recv.tensor)
    ms = time_fn(lambda: ctx.combine(top_i, plan, top_p, T, False))
    gbs = (T * h * 2 + rows * h * 2) / ms / 1e6
    print(f"combine (read T*k rows, write T rows)            {ms:8.3f} ms  {gbs:8.1f} GB/s  {gbs / pk['hbm_gbs']:5.2f} of measured copy bandwidth", flush=True)
    f1 = 2.0 * rows * h * 2 * inter
    ms = time_fn(lambda: ctx.grouped(xp, w1, True, plan))
    print(f"gate_up grouped tcgen05 [{rows}x{h}]x[{h}x{2 * inter}]  {ms:8.3f} ms  {f1 / ms / 1e9:7.1f} TFLOP/s  {f1 / ms / 1e9 / pk['bf16_tflops']:5.2f} of measured peak (useful rows)", flush=True)
    # library path: rows grouped without padding
    order = torch.argsort(top_i.reshape(-1).long(), stable=True)
    xs = x.index_select(0, order // k)
    offs = torch.cumsum(counts, 0).to(torch.int32)
    if hasattr(torch, "_grouped_mm"):
        ms = time_fn(lambda: torch._grouped_mm(xs, w1, offs=offs))
        print(f"gate_up grouped library                          {ms:8.3f} ms  {f1 / ms / 1e9:7.1f} TFLOP/s", flush=True)
    gu = ctx.grouped(xp, w1, True, plan)
    a = native.swiglu_fwd(gu)
    f2 = 2.0 * rows * inter * h
    ms = time_fn(lambda: ctx.grouped(a, w2, True, plan))
    print(f"down grouped tcgen05                             {ms:8.3f} ms  {f2 / ms / 1e9:7.1f} TFLOP/s  {f2 / ms / 1e9 / pk['bf16_tflops']:5.2f} of measured peak", flush=True)
    dy = torch.randn(cap, h, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda: ctx.grouped(dy, w2, False, plan))
    print(f"down dgrad grouped tcgen05                       {ms:8.3f} ms  {f2 / ms / 1e9:7.1f} TFLOP/s  {f2 / ms / 1e9 / pk['bf16_tflops']:5.2f} of measured peak", flush=True)
    w2.main_grad = torch.zeros(E, inter, h, device="cuda", dtype=torch.float32)
    ms = time_fn(lambda: ctx.grouped_wgrad(a, dy, w2, plan))
    print(f"down wgrad grouped tcgen05 (+= fp32)             {ms:8.3f} ms  {f2 / ms / 1e9:7.1f} TFLOP/s  {f2 / ms / 1e9 / pk['bf16_tflops']:5.2f} of measured peak", flush=True)
    torch.cuda.synchronize()
    ctx.check()


def bench_fp8():
    """Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4, 1x128 / 128x128 scales promoted in fp32) on Llama-3-8B shapes, against the
    in-tree and library bf16 GEMMs of the same shape."""
    from nanotron_b200.fp8.quantize import quantize_1x128, quantize_128x128_reference
    from nanotron_b200.ops import native, native_gemm as g

    native.lib()
    peak = _peaks()["bf16_tflops"]
    for name, M, N, K in [("qkv", 8192, 6144, 4096), ("gate_up", 8192, 28672, 4096), ("down", 8192, 4096, 14336)]:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        xq = quantize_1x128(x)
        wq = quantize_128x128_reference(w)
        flops = 2.0 * M * N * K
        ms8 = time_fn(lambda: native.gemm_fp8_blockscaled(xq, wq, epi_warps=8))
        ms8b = time_fn(lambda: native.gemm_fp8_blockscaled(xq, wq, epi_warps=16))
        g.check_status("cuda")
        ms16 = time_fn(lambda: torch.nn.functional.linear(x, w))
        msq = time_fn(lambda: quantize_1x128(x))
        print(f"{name:8s} M={M} N={N} K={K}  fp8 tcgen05 {ms8:7.3f} ms {flops / ms8 / 1e9:7.1f} TFLOP/s ({flops / ms8 / 1e9 / peak:4.2f} of measured bf16 peak; 16 promotion warps: {ms8b:7.3f} ms) | "
              f"library bf16 {ms16:7.3f} ms {flops / ms16 / 1e9:7.1f} TFLOP/s | 1x128 quantise of x {msq:6.3f} ms", flush=True)
        del x, w, xq, wq
        torch.cuda.empty_cache()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if what == "gemm":
        bench_gemm(small="--small" in sys.argv)
    elif what == "gemm-split":
        bench_gemm_split()
    elif what == "elementwise":
        bench_elementwise()
    elif what == "fp8":
        bench_fp8()
    elif what == "moe":
        bench_moe()
    elif what == "attention":
        from bench_attention import main

        main()
