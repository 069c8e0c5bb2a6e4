"""Throughput of the fused compute + collective kernels against their rooflines and against the NCCL + library path.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 tools/bench_fused.py [tp] [dp] [ep] [cp]

Every number is CUDA-event time on the launching stream, 3 warm-up + 10 timed iterations, maximum over ranks.
Roofline of a fused kernel = the slower of (FLOPs / measured GEMM peak) and (bytes that must cross NVLink per GPU / 770 GB/s,
the measured peer-copy bandwidth per direction); for the optimizer step also local HBM bytes / measured copy bandwidth.
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import json

import torch
import torch.distributed as tdist

NVLINK_GBS = 770.0


def _peaks():
    for p in (os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "MEASURED_PEAKS.json"),):
        if os.path.exists(p):
            d = json.load(open(p))
            return {"bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "hbm_gbs": float(d.get("hbm_gbs", 6650.0))}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}


def timed(fn, n_warm=3, n_iter=10) -> float:
    """Milliseconds per call, maximum over ranks."""
    for _ in range(n_warm):
        fn()
    tdist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n_iter):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / n_iter], device="cuda")
    tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    return float(t)


def say(rank, msg):
    if rank == 0:
        print(msg, flush=True)


def bench_tp(group, rank, world, pk):
    from nanotron_b200.ops import tp_fused

    ctx = tp_fused.get_context(group)
    assert ctx is not None, "fused tensor-parallel context unavailable"
    T, h, ffn = 8192, 4096, 14336  # Llama-3-8B layer, 2 x 4096 tokens, sequence-parallel shards of T / tp rows
    rows = T // world
    x = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16)
    w_col = torch.randn(2 * ffn // world, h, device="cuda", dtype=torch.bfloat16) * 0.02
    a = torch.randn(T, ffn // world, device="cuda", dtype=torch.bfloat16)
    w_row = torch.randn(h, ffn // world, device="cuda", dtype=torch.bfloat16) * 0.02
    gathered = torch.empty(T, h, device="cuda", dtype=torch.bfloat16)
    out_rs = torch.empty(rows, h, device="cuda", dtype=torch.bfloat16)

    def nccl_ag_gemm():
        tdist.all_gather_into_tensor(gathered, x, group=group)
        return torch.nn.functional.linear(gathered, w_col)

    def nccl_gemm_rs():
        tdist.reduce_scatter_tensor(out_rs, torch.nn.functional.linear(a, w_row), group=group)

    from nanotron_b200.ops import native_gemm

    link_bytes = (world - 1) / world * T * h * 2
    f1 = 2.0 * T * (2 * ffn // world) * h
    f2 = 2.0 * T * h * (ffn // world)
    ms_n1, ms_n2 = timed(nccl_ag_gemm), timed(nccl_gemm_rs)
    for variant in ("pair", "single"):  # CTA-pair kernel (default) and one-CTA kernel
        native_gemm.set_variant(variant)
        ms_f = timed(lambda: ctx.all_gather_gemm(x, w_col, b_mn=False))
        roof = max(f1 / (pk["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        say(rank, f"tp{world} all-gather->GEMM   [{T}x{h}]x[{h}x{2 * ffn // world}]  fused ({variant}) {ms_f:7.3f} ms | NCCL+library {ms_n1:7.3f} ms | roofline {roof:6.3f} ms -> {roof / ms_f:4.2f} of roofline")
        ms_f = timed(lambda: ctx.gemm_reduce_scatter(a, w_row, b_mn=False))
        roof = max(f2 / (pk["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        say(rank, f"tp{world} GEMM->reduce-scatter [{T}x{ffn // world}]x[{ffn // world}x{h}]  fused ({variant}) {ms_f:7.3f} ms | NCCL+library {ms_n2:7.3f} ms | roofline {roof:6.3f} ms -> {roof / ms_f:4.2f} of roofline")
    native_gemm.set_variant("pair")
    ctx.alloc.check()


def bench_dp(group, rank, world, pk):
    from nanotron_b200.ops import native
    from nanotron_b200.parallel.symm import SymmetricAllocator

    L = native.lib()
    alloc = SymmetricAllocator(group)
    total = 1 << 30  # 1 Gi parameters: 4 GiB of fp32 gradients, 2 GiB of bf16 parameters per rank
    n = total // world
    start = rank * n
    grads = alloc.zeros(total, torch.float32)
    params = alloc.zeros(total, torch.bfloat16)
    grads.tensor.normal_(std=0.01)
    p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    partials = torch.empty(L.ntb_dp_num_partials(), dtype=torch.float32, device="cuda")
    sumsq = torch.zeros(1, device="cuda")
    seg_end = torch.tensor([n], dtype=torch.int64, device="cuda")
    seg_lr = torch.tensor([1e-4], device="cuda")
    seg_wd = torch.tensor([0.1], device="cuda")
    g_shard = grads.tensor[start : start + n]

    def fused():
        s = torch.cuda.current_stream().cuda_stream
        alloc.barrier()
        native._check(L.ntb_dp_reduce_scatter(grads.ptrs, rank, world, start, n, 1.0 / world, 0, partials.data_ptr(), sumsq.data_ptr(), s), "dp_reduce_scatter")
        native._check(L.ntb_dp_adamw_allgather(p.data_ptr(), g_shard.data_ptr(), m.data_ptr(), v.data_ptr(), params.ptrs, rank, world, start, n, seg_end.data_ptr(),
                                               seg_lr.data_ptr(), seg_wd.data_ptr(), 1, 0.9, 0.95, 1e-8, 0.1, 0.05, None, s), "dp_adamw_allgather")
        alloc.barrier()

    rs_out = torch.empty(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    seg_end2 = seg_end.clone()

    def nccl():
        tdist.reduce_scatter_tensor(rs_out, grads.tensor, op=tdist.ReduceOp.AVG, group=group)
        native.sumsq(rs_out)
        native.adamw_flat(p, rs_out, m, v, p16, seg_end2, seg_lr, seg_wd, 0.9, 0.95, 1e-8, 1.0)
        tdist.all_gather_into_tensor(params.tensor, p16, group=group)

    ms_f = timed(fused, n_iter=5)
    ms_n = timed(nccl, n_iter=5)
    # two dependent phases (the clip coefficient needs the norm of the fully reduced gradient before any weight moves):
    #   reduce-scatter: (world - 1) * n * 4 B over NVLink | own slice read + reduced write in HBM
    #   AdamW + all-gather: p, g, m, v read + p, m, v written + bf16 copy in HBM | (world - 1) * n * 2 B over NVLink
    t_rs = max((world - 1) * n * 4 / (NVLINK_GBS * 1e6), n * 4 * 2 / (pk["hbm_gbs"] * 1e6))
    t_opt = max(n * (16 + 12 + 2) / (pk["hbm_gbs"] * 1e6), (world - 1) * n * 2 / (NVLINK_GBS * 1e6))
    roof = t_rs + t_opt
    say(rank, f"dp{world} reduce-scatter + AdamW + all-gather, {total / 2**30:.0f} Gi parameters  fused {ms_f:7.3f} ms | NCCL + kernels {ms_n:7.3f} ms | roofline {roof:6.3f} ms -> {roof / ms_f:4.2f} of roofline")
    alloc.check()


def bench_ep(group, rank, world, pk):
    from nanotron_b200.ops import moe_fused

    T, E, k, h, inter = 8192, 64, 4, 2048, 1408
    torch.manual_seed(rank)
    x = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    probs = torch.softmax(torch.randn(T, E, device="cuda"), -1)
    top_p, top_i = torch.topk(probs, k, dim=-1)
    top_p, top_i = top_p.float().contiguous(), top_i.to(torch.int32).contiguous()
    counts = torch.bincount(top_i.reshape(-1), minlength=E).to(torch.int32)
    ctx = moe_fused.get_context(group, h, T, k, E)
    plan = ctx.make_plan(counts, top_i)
    ms_d = timed(lambda: ctx.dispatch(x, top_i, plan, None, zero_pad=True))
    ctx.ybuf.tensor.copy_(ctx.recv.tensor)
    ctx.barrier()

    def comb():
        ctx.barrier()
        ctx.combine(top_i, plan, top_p, T, False)

    ms_c = timed(comb)
    link = (world - 1) / world * T * k * h * 2  # rows whose expert lives on another GPU
    hbm = T * h * 2 + T * k * h * 2
    roof = max(link / (NVLINK_GBS * 1e6), hbm / (pk["hbm_gbs"] * 1e6))
    say(rank, f"ep{world} dispatch (permute + all-to-all in one kernel + barrier) {ms_d:7.3f} ms | combine {ms_c:7.3f} ms | roofline {roof:6.3f} ms -> {roof / ms_d:4.2f} / {roof / ms_c:4.2f} of roofline")
    # reference: NCCL all-to-all of the same volume with equal splits (no permutation work included)
    send = torch.randn(T * k, h, device="cuda", dtype=torch.bfloat16)
    recv = torch.empty_like(send)
    ms_n = timed(lambda: tdist.all_to_all_single(recv, send, group=group))
    say(rank, f"ep{world} NCCL all_to_all_single of the same volume (equal splits, no permute) {ms_n:7.3f} ms")
    ctx.check()


def bench_cp(group, rank, world, pk):
    from nanotron_b200 import ops
    from nanotron_b200.parallel.context_parallel import fused_ring
    from nanotron_b200.parallel.context_parallel.ring_attention import ring_attention

    B, Hq, Hkv, D = 1, 32, 8, 128
    S = 8192 * world  # 8192 local tokens per GPU (Llama-3-8B heads)
    chunk = S // (2 * world)
    T = 2 * chunk
    torch.manual_seed(rank)
    q, k, v = (torch.randn(T, h, D, device="cuda").to(torch.bfloat16).requires_grad_(True) for h in (Hq, Hkv, Hkv))
    g = torch.randn(T, Hq, D, device="cuda").to(torch.bfloat16)
    pos = torch.zeros(B, T, dtype=torch.long, device="cuda")

    def fused():
        out = fused_ring.fused_ring_attention(q, k, v, group, batch=B)
        out.backward(g)

    def nccl():
        ops.set_attention("auto")
        out = ring_attention(q, k, v, cp_pg=group, causal=True, variant="allgather", position_ids=pos)
        out.backward(g)

    ms_f = timed(fused, n_iter=5)
    ms_n = timed(nccl, n_iter=5)
    # causal attention of this rank's 2 chunks against everything before them: forward 4 * q * keys * D per head, backward 2.5x
    keys = sum((c + 1) * chunk for c in (rank, 2 * world - 1 - rank))
    flops = 3.5 * 4.0 * chunk * (keys - chunk / 2.0) * Hq * D / 1.0
    t = torch.tensor([flops], device="cuda")
    tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    link = (world - 1) / world * S * Hkv * D * 2 * 2 * 3  # K and V read in forward and backward, fp32-sized dK / dV traffic about the same again
    roof = max(float(t) / (pk["bf16_tflops"] * 1e9), link / (NVLINK_GBS * 1e6))
    say(rank, f"cp{world} causal attention fwd+bwd, seq {S} ({T} tokens per GPU)  in-kernel KV exchange {ms_f:7.3f} ms | NCCL all-gather + library attention {ms_n:7.3f} ms | roofline {roof:6.3f} ms -> {roof / ms_f:4.2f} of roofline")
    fused_ring.get_context(group, T, Hkv).alloc.check()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    tdist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    group = tdist.group.WORLD
    pk = _peaks()
    what = sys.argv[1:] or ["tp", "dp", "ep", "cp"]
    for name, fn in (("tp", bench_tp), ("dp", bench_dp), ("ep", bench_ep), ("cp", bench_cp)):
        if name in what:
            fn(group, rank, world, pk)
            torch.cuda.empty_cache()
    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
