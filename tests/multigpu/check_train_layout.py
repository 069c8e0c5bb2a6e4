"""Run with torchrun on tp * pp * dp GPUs: trains a small Llama (head dim 128, so every in-tree kernel runs) for a few steps under the given
layout on fixed data with layout-independent initial weights and writes the loss curve to ``--out``.  Two runs with different layouts
(for instance one GPU, then ``--pp 2`` on two) must produce the same curve up to bf16 reduction-order noise; ``--expect`` compares
with a curve written earlier and prints ``LAYOUT_OK``.

    python tests/multigpu/check_train_layout.py --out /tmp/base.pt
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 tests/multigpu/check_train_layout.py --pp 2 --expect /tmp/base.pt
"""
import argparse
import os
import sys
import zlib

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def name_seeded_init(model):
    """Values depend only on the parameter's canonical name and the element's position in the unsharded tensor."""
    with torch.no_grad():
        for name, p in model.get_named_params_with_correct_tied():
            shape = tuple(p.get_sharded_info().unsharded_shape) if p.is_sharded else tuple(p.shape)
            g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
            full = torch.randn(shape, generator=g, dtype=torch.float32) * 0.02
            if "layernorm" in name or "layer_norm" in name:
                full = 1.0 + full
            if p.is_sharded:
                for sp in p.get_sharded_info().local_global_slices_pairs:
                    p[sp.local_slices] = full[sp.global_slices].to(device=p.device, dtype=p.dtype)
            else:
                p.copy_(full.to(device=p.device, dtype=p.dtype))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--engine", default="1f1b")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--out", default=None)
    ap.add_argument("--expect", default=None)
    ap.add_argument("--tol", type=float, default=0.05)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--keep-gathered", action="store_true", help="tp_recompute_allgather off: column linears keep the gathered activations for their backward")
    args = ap.parse_args()
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1"), os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"), os.environ.setdefault("MASTER_PORT", "29741")
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    import nanotron_b200.distributed as dist
    from helpers import make_config, tiny_llama_config
    from nanotron_b200 import ops
    from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer
    from nanotron_b200.trainer import DistributedTrainer as Base

    class Trainer(Base):
        def _load_model_checkpoint(self, model):
            name_seeded_init(model)
            return model

    seq, total_mbs, vocab = 512, 4, 4096
    mc = tiny_llama_config(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, vocab_size=vocab, max_position_embeddings=seq)
    cfg = make_config(mc, tp=args.tp, pp=args.pp, dp=args.dp, seq=seq, mbs=1, accum=total_mbs // args.dp, steps=args.steps, dtype=args.dtype, lr=1e-3,
                      tp_mode="reduce_scatter" if args.tp > 1 else "all_reduce", async_tp=args.tp > 1, pp_engine=args.engine, zero=1 if args.dp > 1 else 0)
    if args.keep_gathered:
        cfg.parallelism.tp_recompute_allgather = False
    t = Trainer(cfg)
    t.prepare_training()
    ctx = t.parallel_context
    dev = ctx.device
    pp_rank, dp_rank = dist.get_rank(ctx.pp_pg), dist.get_rank(ctx.dp_pg)
    first, last = t.unwrapped_model.input_pp_rank, t.unwrapped_model.output_pp_rank
    g = torch.Generator().manual_seed(1234)
    losses = []
    n0 = ops.native_launches()
    for _ in range(args.steps):
        tokens = torch.randint(0, vocab, (total_mbs, seq + 1), generator=g)
        per = total_mbs // args.dp
        mine = tokens[dp_rank * per : (dp_rank + 1) * per]
        batches = []
        for i in range(per):
            row = mine[i : i + 1]
            b = {}
            b["input_ids"] = row[:, :-1].contiguous().to(dev) if pp_rank == first else TensorPointer(first)
            b["input_mask"] = torch.ones(1, seq, dtype=torch.bool, device=dev) if pp_rank == first else TensorPointer(first)
            b["label_ids"] = row[:, 1:].contiguous().to(dev) if pp_rank == last else TensorPointer(last)
            b["label_mask"] = torch.ones(1, seq, dtype=torch.bool, device=dev) if pp_rank == last else TensorPointer(last)
            batches.append(b)
        _, loss, _ = t.training_step(iter(batches))
        t.iteration_step += 1
        if isinstance(loss, torch.Tensor):
            losses.append(float(loss))
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    launches = ops.native_launches() - n0
    if dist.get_rank(ctx.world_pg) == t.logger_ranks[0]:
        print(f"layout tp={args.tp} pp={args.pp} dp={args.dp} engine={args.engine}: losses {[round(x, 4) for x in losses]} in-tree launches {launches}", flush=True)
        assert (launches > 0 or not torch.cuda.is_available()) and len(losses) == args.steps
        if args.out:
            torch.save(losses, args.out)
        if args.expect:
            exp = torch.load(args.expect)
            for a, b in zip(losses, exp):
                assert abs(a - b) < args.tol, (losses, exp)
            print("LAYOUT_OK", flush=True)
    dist.barrier(ctx.world_pg)
    ctx.destroy()


if __name__ == "__main__":
    main()
