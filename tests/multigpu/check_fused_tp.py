"""Run with torchrun on 2+ GPUs: fused all-gather->GEMM and GEMM->reduce-scatter kernels against the NCCL + library path,
first as bare ops (forward and backward), then inside a sequence-parallel tiny Llama training run.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_fused_tp.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from helpers import dummy_dataloader, make_config, tiny_llama_config  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def check_ops(ctx):
    import nanotron_b200.distributed as dist
    from nanotron_b200.ops import tp_fused
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
    from nanotron_b200.parallel.tensor_parallel.functional import column_linear, row_linear

    tp, rank = ctx.tp_pg.size(), dist.get_rank(ctx.tp_pg)
    torch.manual_seed(1234 + rank)
    M, K, N = 512, 1024, 1536
    results = {}
    for fused in (False, True, "overlapped push"):  # the last: this rank's push on a side stream beside the GEMM
        tp_fused.ENABLED = bool(fused)
        tp_fused.OVERLAP_PUSH = fused == "overlapped push"
        tp_fused._CONTEXTS.clear()
        torch.manual_seed(7 + rank)
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w_col = (torch.randn(N // tp, K, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
        w_row = (torch.randn(K, N // tp, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
        h = column_linear(x, w_col, None, ctx.tp_pg, TensorParallelLinearMode.REDUCE_SCATTER, async_communication=True)
        y = row_linear(torch.tanh(h), w_row, None, ctx.tp_pg, TensorParallelLinearMode.REDUCE_SCATTER, async_communication=True)
        g = torch.randn_like(y)
        y.backward(g)
        torch.cuda.synchronize()
        results[fused] = (h.detach(), y.detach(), x.grad.detach(), w_col.grad.detach(), w_row.grad.detach())
        if fused:
            c = tp_fused.get_context(ctx.tp_pg)
            assert c is not None, "fused context was not created"
            c.alloc.check()
            assert c.ag_calls >= 2 and c.rs_calls >= 2, (c.ag_calls, c.rs_calls)  # forward + backward of each linear went through the fused kernels
            if rank == 0:
                print(f"  fused kernel calls: all-gather(+GEMM) {c.ag_calls}, GEMM+reduce-scatter {c.rs_calls}")
    tp_fused.OVERLAP_PUSH = False
    names = ["column out", "row out", "dx", "dW column", "dW row"]
    for key in (True, "overlapped push"):
        for n, a, b in zip(names, results[key], results[False]):
            e = rel(a, b)
            if rank == 0:
                print(f"  {n:12s} rel err fused{'' if key is True else ' (' + key + ')'} vs nccl = {e:.3e}")
            assert e < 2e-2, (n, e)


def train(fused: bool, steps=4):
    from nanotron_b200.ops import tp_fused
    from nanotron_b200.trainer import DistributedTrainer

    tp_fused.ENABLED = fused
    tp_fused._CONTEXTS.clear()
    world = int(os.environ["WORLD_SIZE"])
    mc = tiny_llama_config(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=1024)
    cfg = make_config(mc, tp=world, seq=256, mbs=2, steps=steps, dtype="bfloat16", tp_mode="reduce_scatter", async_tp=True, lr=1e-3)
    torch.manual_seed(0)
    t = DistributedTrainer(cfg)
    t.prepare_training()
    dl = dummy_dataloader(t)
    losses = []
    for _ in range(steps):
        _, loss, _ = t.training_step(dl)
        t.iteration_step += 1
        losses.append(float(loss))
    if fused:
        c = tp_fused.get_context(t.parallel_context.tp_pg)
        assert c is not None and c.ag_calls > 0 and c.rs_calls > 0, "training did not go through the fused tensor-parallel kernels"
    return losses, t.parallel_context


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    base, ctx = train(False)
    fused, _ = train(True)
    if rank == 0:
        print("nccl  losses", ["%.4f" % l for l in base])
        print("fused losses", ["%.4f" % l for l in fused])
    assert all(abs(a - b) < 3e-2 for a, b in zip(base, fused)), (base, fused)
    from nanotron_b200.ops import native_gemm

    for variant in ("pair", "single"):  # the fused modes exist on both in-tree GEMM kernels
        native_gemm.set_variant(variant)
        if rank == 0:
            print(f"GEMM kernel: {variant}")
        check_ops(ctx)
    native_gemm.set_variant("pair")
    if rank == 0:
        print("FUSED_TP_OK")
    import torch.distributed as tdist

    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
