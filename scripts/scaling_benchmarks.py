#!/usr/bin/env python
"""Sweep parallel layouts and tabulate throughput (capability parity: reference scripts/scaling_benchmarks.py, which generates
configs and slurm jobs over dp / tp / pp / batch-accumulation grids and collects tokens/s and MFU into a CSV).

Two modes:

    # one node, now: one torchrun of bench.py per layout, JSON lines -> CSV
    python scripts/scaling_benchmarks.py --gpus 8 --model llama3-8b --out results/scaling.csv [--layouts dp8 dp4tp2 dp2tp4 tp8 dp4pp2]

    # any number of nodes, through slurm: one training config + one sbatch script per (model size, layout); the jobs run
    # run_train.py under NANOTRON_BENCHMARK=1, which appends a row to --benchmark-csv at iteration 4 and exits
    python scripts/scaling_benchmarks.py generate --sizes 1B 8B --nodes 1 2 --configs-dir bench/configs --scripts-dir bench/scripts \
        --benchmark-csv bench/results.csv [--submit] [--limit 0:10] [--partition P] [--time 00:40:00]

In the first mode each layout is one ``torchrun`` of ``bench.py`` (same timing rules: CUDA events, barrier + synchronize, max over
ranks).  A layout that fails or runs out of memory is recorded with its exit code and the sweep continues.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def parse_layout(name: str):
    parts = dict(dp=1, tp=1, pp=1)
    for key, val in re.findall(r"(dp|tp|pp)(\d+)", name):
        parts[key] = int(val)
    return parts


def default_layouts(gpus: int):
    out = []
    tp = 1
    while tp <= gpus:
        pp = 1
        while tp * pp <= gpus:
            dp = gpus // (tp * pp)
            if dp * tp * pp == gpus:
                out.append(f"dp{dp}tp{tp}pp{pp}")
            pp *= 2
        tp *= 2
    return out


def run_layout(args, layout: str, port: int):
    p = parse_layout(layout)
    world = p["dp"] * p["tp"] * p["pp"]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(REPO, "bench.py"), "--gpus", str(world), "--steps", str(args.steps), "--warmup", str(args.warmup), "--model", args.model, "--seq", str(args.seq),
           "--mbs", str(args.mbs), "--accum", str(args.accum), "--tp", str(p["tp"]), "--pp", str(p["pp"])]
    if args.recompute:
        cmd.append("--recompute")
    if world == 1:
        cmd = [sys.executable] + cmd[cmd.index(os.path.join(REPO, "bench.py")):]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=args.timeout, cwd=REPO)
    line = next((l for l in reversed(r.stdout.splitlines()) if l.startswith("{")), None)
    row = {"layout": layout, "returncode": r.returncode}
    if line:
        d = json.loads(line)
        row.update(tokens_per_s=d["value"], tokens_per_s_per_gpu=d["tokens_per_sec_per_gpu"], ms_per_step=d["ms_per_step"], model_tflops_per_gpu=d["model_tflops_per_gpu"],
                   mfu=d["mfu_of_measured_sustained_peak"], peak_mem_gb=d.get("peak_mem_gb"), parallelism=d["config"]["parallelism"], sm_mhz=(d.get("clocks") or {}).get("sm_mhz"))
    else:
        row["error"] = (r.stderr or r.stdout)[-300:].replace("\n", " ")
    return row


# ---------------------------------------------------------------------------- slurm sweep generation
# name -> (layers, hidden, heads, kv heads, ffn, vocab); the sizes the reference's published sweep uses (scripts/scaling_benchmarks.py:303-311)
MODEL_SIZES = {
    "1B": (16, 2048, 32, 8, 8192, 131072),
    "3B": (28, 3072, 32, 8, 8192, 131072),
    "8B": (32, 4096, 32, 8, 14336, 131072),
    "70B": (80, 8192, 64, 8, 28672, 131072),
}


def estimate_num_params(layers: int, hidden: int, heads: int, kv_heads: int, ffn: int, vocab: int, tie_word_embeddings: bool) -> int:
    """Embedding (+ head unless tied) + per layer: q and o projections, k and v projections of the kv heads, three ffn matrices."""
    emb = vocab * hidden * (1 if tie_word_embeddings else 2)
    attn = 2 * hidden * hidden + 2 * hidden * hidden * kv_heads // heads
    return emb + layers * (attn + 3 * hidden * ffn)


def _human(n: float) -> str:
    for unit, div in (("T", 1e12), ("B", 1e9), ("M", 1e6)):
        if n >= div:
            return f"{n / div:.3g}{unit}"
    return str(int(n))


def layouts_for(world: int, max_tp: int = 8, max_pp: int = 16):
    """Every (dp, tp, pp) with dp * tp * pp == world, tp a power of two inside a node, pp a power of two."""
    out = []
    tp = 1
    while tp <= min(max_tp, world):
        pp = 1
        while tp * pp <= world and pp <= max_pp:
            if world % (tp * pp) == 0:
                out.append((world // (tp * pp), tp, pp))
            pp *= 2
        tp *= 2
    return out


def create_config(size: str, dp: int, tp: int, pp: int, batch_accum: int, seq_len: int, micro_batch_size: int, zero_stage: int, benchmark_csv: str, profile: bool = False):
    """Full training config of one experiment (dummy data, sequence-parallel tensor parallelism with fused communication)."""
    sys.path.insert(0, REPO)
    import nanotron_b200.config as c

    layers, hidden, heads, kv, ffn, vocab = MODEL_SIZES[size]
    tie = ffn < 10_000  # the small models of the sweep tie their embeddings
    n = estimate_num_params(layers, hidden, heads, kv, ffn, vocab, tie)
    run = f"{_human(n)}_dp{dp}_tp{tp}_pp{pp}_acc{batch_accum}_mbs{micro_batch_size}_seq{seq_len}_zero{zero_stage}_gqa{kv}" + ("_prof" if profile else "")
    mc = c.LlamaConfig(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv, vocab_size=vocab,
                       max_position_embeddings=seq_len, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=tie)
    return c.Config(
        general=c.GeneralArgs(project="scaling_benchmarks", run=run, seed=42, benchmark_csv_path=benchmark_csv),
        parallelism=c.ParallelismArgs(dp=dp, pp=pp, tp=tp, pp_engine="1f1b", tp_mode="reduce_scatter", tp_linear_async_communication=tp > 1),
        model=c.ModelArgs(model_config=mc, init_method=c.RandomInit(std=0.02), dtype="bfloat16"),
        tokenizer=c.TokenizerArgs(),
        checkpoints=c.CheckpointsArgs(checkpoints_path=f"checkpoints/{run}", checkpoint_interval=10**6, save_final_state=False),
        logging=c.LoggingArgs(log_level="info", log_level_replica="warning", iteration_step_info_interval=1),
        tokens=c.TokensArgs(sequence_length=seq_len, train_steps=10 if profile else 100, micro_batch_size=micro_batch_size, batch_accumulation_per_replica=batch_accum),
        optimizer=c.OptimizerArgs(
            optimizer_factory=c.AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True), zero_stage=zero_stage, weight_decay=0.01,
            clip_grad=1.0, accumulate_grad_in_fp32=True, learning_rate_scheduler=c.LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2, lr_decay_style="cosine", min_decay_lr=3e-5),
        ),
        data_stages=[c.DatasetStageArgs(name="bench", start_training_step=1, data=c.DataArgs(dataset=None, seed=42, num_loading_workers=0))],
        profiler=c.ProfilerArgs(profiler_export_path="./tb_logs") if profile else None,
    ), n


SLURM_TEMPLATE = """#!/bin/bash
#SBATCH --job-name={job_name}
#SBATCH --nodes={nodes}
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node={gpus_per_node}
#SBATCH --exclusive
#SBATCH --partition={partition}
#SBATCH --time={time}
#SBATCH --output={logs_dir}/%x-%j.out
set -euo pipefail
export NANOTRON_BENCHMARK=1
export CUDA_DEVICE_MAX_CONNECTIONS=1
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))
srun --wait=0 --kill-on-bad-exit=1 bash -c 'python -m torch.distributed.run --nnodes={nodes} --nproc-per-node={gpus_per_node} --node-rank=$SLURM_PROCID \
    --master-addr $MASTER_ADDR --master-port $MASTER_PORT --max-restarts 0 {repo}/run_train.py --config-file {config_path}'
"""


def generate(args):
    """Write one config + one sbatch script per experiment, the experiment table as CSV, and optionally submit the jobs."""
    os.makedirs(args.configs_dir, exist_ok=True)
    os.makedirs(args.scripts_dir, exist_ok=True)
    os.makedirs(args.logs_dir, exist_ok=True)
    experiments = []
    for size in args.sizes:
        layers = MODEL_SIZES[size][0]
        for nodes in args.nodes:
            world = nodes * args.gpus_per_node
            for dp, tp, pp in layouts_for(world, max_tp=args.gpus_per_node):
                if pp > layers or MODEL_SIZES[size][3] % tp:
                    continue  # more stages than layers, or kv heads not divisible by tp
                # global batch of about args.gbs_tokens tokens: accumulation makes up what dp * mbs does not cover
                accum = max(1, args.gbs_tokens // (args.seq * args.mbs * dp))
                if pp > 1 and accum < pp - 1:
                    continue  # 1F1B needs at least pp - 1 micro-batches
                for zero in ((0, 1) if dp > 1 else (0,)):
                    experiments.append(dict(size=size, nodes=nodes, dp=dp, tp=tp, pp=pp, batch_accum=accum, seq_len=args.seq, mbs=args.mbs, zero_stage=zero))
    if args.limit:
        lo, _, hi = args.limit.partition(":")
        experiments = experiments[(int(lo) if lo else None) : (int(hi) if hi else None)] if ":" in args.limit else experiments[: int(args.limit)]
    rows = []
    for e in experiments:
        cfg, n_params = create_config(e["size"], e["dp"], e["tp"], e["pp"], e["batch_accum"], e["seq_len"], e["mbs"], e["zero_stage"], args.benchmark_csv, profile=args.profile)
        name = cfg.general.run
        config_path = os.path.abspath(os.path.join(args.configs_dir, f"{name}.yaml"))
        cfg.save_as_yaml(config_path)
        script_path = os.path.join(args.scripts_dir, f"{name}.sh")
        with open(script_path, "w") as fo:
            fo.write(SLURM_TEMPLATE.format(job_name=f"bench_{name}", nodes=e["nodes"], gpus_per_node=args.gpus_per_node, partition=args.partition, time=args.time,
                                           logs_dir=os.path.abspath(args.logs_dir), repo=REPO, config_path=config_path))
        os.chmod(script_path, 0o755)
        job_id = ""
        if args.submit:
            r = subprocess.run(["bash" if args.use_bash else "sbatch", script_path], capture_output=True, text=True)
            job_id = (r.stdout.strip().split() or [""])[-1] if r.returncode == 0 else f"failed:{r.returncode}"
        rows.append(dict(e, run=name, num_params=n_params, config=config_path, script=script_path, job_id=job_id))
    table = os.path.join(args.configs_dir, "experiments.csv")
    with open(table, "w", newline="") as fo:
        w = csv.DictWriter(fo, fieldnames=list(rows[0].keys()) if rows else ["run"])
        w.writeheader()
        w.writerows(rows)
    print(f"{len(rows)} experiments: configs in {args.configs_dir}, scripts in {args.scripts_dir}, table {table}")
    return rows


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "generate":
        ap = argparse.ArgumentParser(prog="scaling_benchmarks.py generate")
        ap.add_argument("--sizes", nargs="+", default=["8B"], choices=sorted(MODEL_SIZES))
        ap.add_argument("--nodes", nargs="+", type=int, default=[1])
        ap.add_argument("--gpus-per-node", type=int, default=8)
        ap.add_argument("--seq", type=int, default=4096)
        ap.add_argument("--mbs", type=int, default=1)
        ap.add_argument("--gbs-tokens", type=int, default=1 << 20, help="target tokens per optimizer step")
        ap.add_argument("--configs-dir", default="benchmark/configs")
        ap.add_argument("--scripts-dir", default="benchmark/scripts")
        ap.add_argument("--logs-dir", default="benchmark/logs")
        ap.add_argument("--benchmark-csv", default="benchmark/results.csv")
        ap.add_argument("--partition", default="gpu")
        ap.add_argument("--time", default="00:40:00")
        ap.add_argument("--limit", default=None, help="N or START:END slice of the experiment list")
        ap.add_argument("--profile", action="store_true")
        ap.add_argument("--submit", action="store_true", help="sbatch every generated script")
        ap.add_argument("--use-bash", action="store_true", help="with --submit: run the scripts with bash instead of sbatch")
        generate(ap.parse_args(sys.argv[2:]))
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--accum", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--timeout", type=int, default=1200)
    ap.add_argument("--layouts", nargs="*", default=None, help="e.g. dp8 dp4tp2 dp2tp2pp2 (default: every power-of-two factorisation of --gpus)")
    ap.add_argument("--out", default="scaling.csv")
    args = ap.parse_args()
    layouts = args.layouts or default_layouts(args.gpus)
    rows = []
    for i, layout in enumerate(layouts):
        row = run_layout(args, layout, 29600 + i)
        rows.append(row)
        print(json.dumps(row), flush=True)
    keys = sorted({k for r in rows for k in r}, key=lambda k: (k != "layout", k))
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys)
        w.writeheader()
        w.writerows(rows)
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
