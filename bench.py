#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B pre-training throughput (tokens/s, whole job) on N B200s of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus 8
    python bench.py --impl reference ...      # the unmodified reference installed under baseline/_ref, same layout

What is timed: full training steps (forward, backward, gradient reduction, clipping, AdamW on fp32 masters, bf16
parameter refresh) of a random-init Llama-3-8B (32 layers, hidden 4096, ffn 14336, 32/8 heads, vocab 128256) on
uniform-random tokens: 8 micro-batches of one 4096-token sequence per step, bf16 compute with fp32 gradient accumulation
and fp32 master weights.  Layout by GPU count (``--layout model``, the default; both arms use the same one):

    N = 1: one GPU            N = 2: tp 2            N = 4: tp 4            N = 8: tp 4 x pp 2 (1F1B)

with sequence-parallel tensor parallelism and asynchronous tp communication, the layout the reference's own scaling
benchmark uses for this model class.  The global batch is the same at every N (strong scaling).  ``--layout dp`` instead
replicates the model on every GPU with ZeRO-1 (dp = N, weak scaling: every GPU processes 8 micro-batches); the reference
cannot run that layout for an 8B model (it needs more than the 180 GB of a B200), so it has no reference number.
Timing: CUDA events around exactly K steps, barrier + synchronize on both sides, max over ranks.  The working set
of a step (tens of GB) is far larger than L2, so no explicit L2 flush is done between steps.
A second number ("e2e") times the same steps through ``DistributedTrainer.training_step`` with the inputs built in
pinned host memory and copied to the device every micro-batch, and the loss read back to the host every step.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# reference's published best single-node MFU for its 8.86B model (45.22 % of 989 TFLOPs on H100) expressed as tokens/s/GPU
BASELINE_TOK_S_PER_GPU = 7900.0

MODELS = {
    "llama3-8b": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=4096, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "llama3.2-1b": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=4096, rms_norm_eps=1e-5, tie_word_embeddings=True),
    "tiny": dict(hidden_size=512, intermediate_size=1536, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=4, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096, rms_norm_eps=1e-5, tie_word_embeddings=False),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._proc = None
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            if self._stop.is_set():
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self) -> dict:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                pass
        clocks, reasons, max_mhz = [], set(), None
        for s in self.samples:
            try:
                clocks.append(float(s[0]))
                max_mhz = float(s[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons), "samples": len(clocks)}


# Other target configurations, selected with --config (they set model / batch / layout flags; explicit flags still win):
#   llama3.2-1b-dp8    Llama-3.2-1B, data parallel over all GPUs with ZeRO-1, micro-batch 4, one accumulation step
#   qwen-moe-ep8       Qwen-style MoE (64 experts top-4 + shared expert, aux loss 0.01), expert parallel over all GPUs (on the dp axis), micro-batch 2
#   llama3-8b-cp8-64k  Llama-3-8B at 65536 tokens, context parallel over all GPUs (zig-zag sharding), activation recompute
CONFIGS = {
    "llama3-8b": {},
    "llama3.2-1b-dp8": dict(model="llama3.2-1b", layout="dp", mbs=4, accum=1),
    "qwen-moe-ep8": dict(model="qwen-moe", layout="dp", ep=-1, mbs=2, accum=1),
    "llama3-8b-cp8-64k": dict(model="llama3-8b", cp=-1, seq=65536, mbs=1, accum=1, recompute=True),
}
QWEN_MOE = dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=24, num_attention_heads=16, num_key_value_heads=4, vocab_size=151936, rope_theta=1000000.0,
                max_position_embeddings=4096, rms_norm_eps=1e-6, tie_word_embeddings=False)
QWEN_MOE_EXPERTS = dict(num_experts=64, top_k=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632, enable_shared_expert=True, router_aux_loss_coef=0.01)

MODEL_LAYOUTS = {1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (4, 2)}  # GPUs -> (tp, pp); dp = GPUs / (tp * pp)


def resolve_layout(args, world: int):
    """(tp, pp, dp) of a run: explicit --tp / --pp win, else the layout table (``model``) or pure data parallelism (``dp``)."""
    cp = getattr(args, "cp", 1) or 1
    cp = world if cp < 0 else cp
    if args.tp is not None or args.pp is not None:
        tp, pp = args.tp or 1, args.pp or 1
    elif args.layout == "dp" or cp > 1:
        tp, pp = 1, 1
    else:
        tp, pp = MODEL_LAYOUTS.get(world, (min(world, 4), 1))
    assert world % (tp * pp * cp) == 0, f"world size {world} is not a multiple of tp * pp * cp = {tp * pp * cp}"
    return tp, pp, world // (tp * pp * cp)


def layout_label(tp: int, pp: int, dp: int, zero: int) -> str:
    parts = []
    if dp > 1 or (tp == 1 and pp == 1):
        parts.append(f"dp{dp}" + ("+zero1" if zero else ""))
    if tp > 1:
        parts.append(f"tp{tp}(sequence-parallel, async)")
    if pp > 1:
        parts.append(f"pp{pp}(1f1b)")
    return "x".join(parts)


def build_config(args, world: int):
    import nanotron_b200.config as c

    if args.model == "qwen-moe":
        mc = c.Qwen2Config(moe_config=c.MoEConfig(**QWEN_MOE_EXPERTS), **QWEN_MOE)
    else:
        mc = c.LlamaConfig(**MODELS[args.model])
    if args.layers is not None:
        mc.num_hidden_layers = args.layers  # shortened model for trying a configuration on fewer GPUs: not a benchmark number
    tp, pp, dp = resolve_layout(args, world)
    cp = world // (tp * pp * dp)
    ep = dp if (args.ep or 1) < 0 else (args.ep or 1)
    zero = 1 if (dp > 1 and ep == 1) else 0
    if cp > 1:
        mc.max_position_embeddings = max(mc.max_position_embeddings, args.seq)
    return c.Config(
        general=c.GeneralArgs(project="bench", run="bench", seed=42, ignore_sanity_checks=True),
        parallelism=c.ParallelismArgs(dp=dp, pp=pp, tp=tp, pp_engine="1f1b", tp_mode="reduce_scatter", tp_linear_async_communication=tp > 1, recompute_layer=args.recompute,
                                      # --tp-keep-gathered: column linears keep their gathered input for the backward instead of gathering it again
                                      # (measured on 2 GPUs: 38.65 k against 38.2 - 38.8 k tokens/s, +1 GB: no gain, so gathering again stays the default)
                                      tp_recompute_allgather=not bool(getattr(args, "tp_keep_gathered", False)),
                                      context_parallel_size=cp, expert_parallel_size=ep),
        model=c.ModelArgs(model_config=mc, init_method=c.RandomInit(std=0.02), dtype="bfloat16"),
        tokenizer=c.TokenizerArgs(),
        checkpoints=c.CheckpointsArgs(checkpoints_path="/tmp/ntb_bench_ckpt", checkpoint_interval=10**9, save_final_state=False),
        logging=c.LoggingArgs(log_level="warning", log_level_replica="error", iteration_step_info_interval=10**9),
        tokens=c.TokensArgs(sequence_length=args.seq, train_steps=10**6, micro_batch_size=args.mbs, batch_accumulation_per_replica=args.accum),
        optimizer=c.OptimizerArgs(
            optimizer_factory=c.AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
            zero_stage=zero, weight_decay=0.01, clip_grad=1.0, accumulate_grad_in_fp32=True, overlap_grad_reduce=not args.no_grad_overlap,
            learning_rate_scheduler=c.LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2, lr_decay_style="cosine", min_decay_lr=3e-5),
        ),
        data_stages=[c.DatasetStageArgs(name="bench", start_training_step=1, data=c.DataArgs(dataset=None, seed=42, num_loading_workers=0))],
    )


def run_native(args):
    import torch

    import nanotron_b200.distributed as dist
    from nanotron_b200 import ops
    from nanotron_b200.data.dataloader import dummy_infinite_data_generator
    from nanotron_b200.models.qwen import get_flops
    from nanotron_b200.trainer import DistributedTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1"), os.environ.setdefault("LOCAL_RANK", "0")
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    ops.set_gemm(args.gemm)
    ops.set_attention(args.attention)
    ops.set_linear(args.linear)
    from nanotron_b200.ops import native_gemm

    native_gemm.set_variant(args.gemm_variant)
    cfg = build_config(args, world)
    trainer = DistributedTrainer(cfg)
    trainer.prepare_training()
    ctx = trainer.parallel_context
    mc = trainer.model_config

    def gen(host_pinned: bool):
        return dummy_infinite_data_generator(
            micro_batch_size=args.mbs, sequence_length=args.seq, input_pp_rank=trainer.unwrapped_model.input_pp_rank,
            output_pp_rank=trainer.unwrapped_model.output_pp_rank, vocab_size=mc.vocab_size,
            seed=42, parallel_context=ctx, use_position_ids=args.model == "qwen-moe", host_pinned=host_pinned,
        )()

    def timed(loader, steps, read_loss: bool):
        dist.barrier(ctx.world_pg)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.native_launches()
        start.record()
        last = None
        for _ in range(steps):
            _, loss, _ = trainer.training_step(loader)
            trainer.iteration_step += 1
            if read_loss and isinstance(loss, torch.Tensor):
                last = float(loss.item())  # device -> host read of the step result (pipeline ranks without the loss have none)
            else:
                last = loss
        end.record()
        torch.cuda.synchronize()
        dist.barrier(ctx.world_pg)
        ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=ctx.world_pg)
        return float(ms.item()), ops.native_launches() - launches0, last

    dev_loader, host_loader = gen(False), gen(True)
    timed(dev_loader, args.warmup, read_loss=False)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms, launches, loss = timed(dev_loader, args.steps, read_loss=False)
    clocks = sampler.stop()
    loss_t = loss if isinstance(loss, torch.Tensor) else torch.zeros((), device="cuda")
    loss_t = loss_t.detach().float().reshape(1).clone()
    dist.all_reduce(loss_t, op=dist.ReduceOp.MAX, group=ctx.world_pg)  # ranks that do not hold the loss contribute 0
    loss_val = float(loss_t.item())
    timed(host_loader, 1, read_loss=True)
    e2e_ms, _, _ = timed(host_loader, args.steps, read_loss=True)

    dp = ctx.dp_pg.size()
    tp, pp = ctx.tp_pg.size(), ctx.pp_pg.size()
    tokens_per_step = args.mbs * args.seq * args.accum * dp
    value = tokens_per_step / (ms / args.steps / 1000.0)
    e2e_value = tokens_per_step / (e2e_ms / args.steps / 1000.0)
    ffn = mc.intermediate_size
    if args.model == "qwen-moe":
        # active parameters per token: top-k routed experts + the shared expert (the router itself is negligible)
        ffn = QWEN_MOE_EXPERTS["top_k"] * QWEN_MOE_EXPERTS["moe_intermediate_size"] + QWEN_MOE_EXPERTS["shared_expert_intermediate_size"]
    flops, _ = get_flops(num_layers=mc.num_hidden_layers, hidden_size=mc.hidden_size, num_heads=mc.num_attention_heads, num_key_value_heads=mc.num_key_value_heads, vocab_size=mc.vocab_size, seq_len=args.seq, ffn_hidden_size=ffn, batch_size=1)
    tflops_per_gpu = flops / args.seq * value / world / 1e12
    peaks = {}
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak = peaks.get("bf16_tflops_sustained", 1400.0)
    if rank == 0:
        out = {
            "metric": "Llama-3-8B training tokens/sec (whole job), bf16, seq 4096" if (args.model == "llama3-8b" and args.seq == 4096 and args.layers is None) else f"{args.config} training tokens/sec (whole job), bf16, seq {args.seq}",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak" if dp == world else "strong", "vs_baseline": value / world / BASELINE_TOK_S_PER_GPU if (args.model == "llama3-8b" and args.seq == 4096) else None,
            "dtype": "bf16" if args.linear == "bf16" else "fp8 (block-scaled linears; bf16 elsewhere)", "data": "synthetic uniform-random tokens, random-init weights",
            "tokens_per_sec_per_gpu": value / world, "model_tflops_per_gpu": tflops_per_gpu, "mfu_of_measured_sustained_peak": tflops_per_gpu / peak,
            "loss": loss_val, "impl": "nanotron_b200",
            "config": {
                "model": args.model + (f" (shortened to {args.layers} layers)" if args.layers is not None else ""), "global_batch": args.mbs * args.accum * dp, "seq_len": args.seq, "micro_batch": args.mbs, "grad_accum": args.accum,
                "parallelism": layout_label(tp, pp, dp, 1 if (dp > 1 and ctx.expert_parallel_size == 1) else 0) + (f"xcp{ctx.cp_pg.size()}(zig-zag)" if ctx.cp_pg.size() > 1 else "") + (f"+ep{ctx.expert_parallel_size}(on the dp axis)" if ctx.expert_parallel_size > 1 else ""),
                "tp_linears": "in-tree fused all-gather->GEMM / GEMM->reduce-scatter kernels over NVLink peer memory" if tp > 1 else "n/a",
                "tp_recompute_allgather": (not bool(args.tp_keep_gathered)) if tp > 1 else None,
                "pp_p2p": "NCCL send/recv on one lane per direction, asynchronous" if pp > 1 else "n/a",
                "dp_step": ("in-tree NVLink kernels (reduce-scatter" + (" per layer during the last backward" if (trainer.fused_dp.buckets and not args.no_grad_overlap) else "") + " + AdamW + all-gather)") if getattr(trainer, "fused_dp", None) is not None else "NCCL", "fp32_grad_accum": True, "fp32_master_weights": True, "optimizer": "AdamW", "clip_grad": 1.0,
                "recompute_layer": bool(args.recompute), "l2": "inputs larger than L2 (per-step working set is tens of GB); no explicit flush",
                "gemm": ops._GEMM, "gemm_kernel": args.gemm_variant, "attention": ops._ATTN, "linear": ops.get_linear(),
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": 2 * args.mbs * args.seq * 8 * args.accum, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
        }
        print(json.dumps(out), flush=True)
    dist.barrier(ctx.world_pg)
    ctx.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--config", default="llama3-8b", choices=sorted(CONFIGS), help="target configuration preset (sets --model / --layout / batch flags; flags given explicitly win)")
    ap.add_argument("--model", default=None, choices=sorted(MODELS) + ["qwen-moe"])
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--mbs", type=int, default=None)
    ap.add_argument("--accum", type=int, default=None)
    ap.add_argument("--recompute", action="store_true", default=None)
    ap.add_argument("--tp-keep-gathered", action="store_true", help="tensor-parallel column linears keep the gathered copy of their input for the backward instead of gathering it again")
    ap.add_argument("--no-grad-overlap", action="store_true", help="data-parallel runs: reduce-scatter all gradients after the last backward instead of per layer during it")
    ap.add_argument("--layers", type=int, default=None, help="override the number of layers (for trying a configuration on fewer GPUs; the result is not a benchmark of the named model)")
    ap.add_argument("--cp", type=int, default=None, help="context-parallel size (-1: all GPUs)")
    ap.add_argument("--ep", type=int, default=None, help="expert-parallel size, laid over the dp axis (-1: dp)")
    ap.add_argument("--gemm", default="auto", choices=["auto", "tcgen05", "cublas"], help="auto / tcgen05: every linear-layer product on the in-tree tcgen05 kernels; cublas: library GEMMs (wgrad then needs a separate fp32 add)")
    ap.add_argument("--attention", default="auto", choices=["auto", "native", "sdpa"], help="auto / native: the in-tree tcgen05 flash-attention kernels; sdpa: library attention (comparison runs)")
    ap.add_argument("--linear", default="bf16", choices=["bf16", "fp8"], help="fp8: block-scaled fp8 operands (e4m3 forward, e5m2 gradients) for the linear-layer products")
    ap.add_argument("--gemm-variant", default="pair", choices=["single", "pair"], help="in-tree GEMM kernel: one CTA per 128x256 tile, or CTA pairs (cta_group::2) per 256x256 tile")
    ap.add_argument("--layout", default=None, choices=["model", "dp"], help="model: tp / pp by GPU count (1: none, 2: tp2, 4: tp4, 8: tp4 x pp2), same global batch at every N; dp: data parallel over all GPUs with ZeRO-1")
    ap.add_argument("--tp", type=int, default=None, help="tensor-parallel size (sequence-parallel mode), overrides --layout; dp = gpus / (tp * pp)")
    ap.add_argument("--pp", type=int, default=None, help="pipeline-parallel size (1F1B), overrides --layout")
    args = ap.parse_args()
    defaults = dict(model="llama3-8b", seq=4096, mbs=1, accum=8, recompute=False, cp=1, ep=1, layout="model")
    defaults.update(CONFIGS[args.config])
    for k, v in defaults.items():
        if getattr(args, k) is None:
            setattr(args, k, v)
    if args.impl == "reference":
        from baseline.run_reference import run_reference

        return run_reference(args)
    run_native(args)


if __name__ == "__main__":
    main()
