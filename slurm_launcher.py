#!/usr/bin/env python
"""Builds a training config from command-line presets and submits it to slurm (parity: reference slurm_launcher.py).

    python slurm_launcher.py --run my_run --model 1b --nodes 2 --dp 16 --tp 1 --pp 1 --seq 4096 --mbs 2 --acc 8 --steps 1000 --dry-run

Writes ``<configs-path>/<run>.yaml`` and ``<slurm-scripts-dir>/<run>.slurm``; ``--dry-run`` stops there, otherwise the
script is handed to ``sbatch``.  torchrun is started with ``--max_restarts 0``: recovery is checkpoint + resubmit.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, LRSchedulerArgs, ModelArgs, NanosetDatasetsArgs,
    OptimizerArgs, ParallelismArgs, ProfilerArgs, Qwen2Config, RandomInit, TokenizerArgs, TokensArgs,
)

# (hidden, layers, heads, kv heads, intermediate)
MODEL_SIZES = {
    "160m": (768, 12, 12, 12, 3072),
    "410m": (1024, 24, 16, 16, 4096),
    "1b": (2048, 16, 32, 8, 8192),
    "3b": (3072, 28, 24, 8, 8192),
    "8b": (4096, 32, 32, 8, 14336),
    "70b": (8192, 80, 64, 8, 28672),
    "custom": None,
}


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--run", type=str, default="nanotron", help="run name")
    g = p.add_argument_group("slurm")
    g.add_argument("--gpus-per-node", type=int, default=8)
    g.add_argument("--partition", type=str, default="b200")
    g.add_argument("--qos", type=str, default="normal")
    g.add_argument("--time-limit", type=str, default="24:00:00")
    g.add_argument("--nodes", type=int, default=1)
    g.add_argument("--reservation", type=str, default=None)
    g.add_argument("--dry-run", action="store_true")
    g.add_argument("--show-logs", action="store_true")
    g.add_argument("--env", type=str, default=None, help="conda/venv activate line")
    m = p.add_argument_group("model")
    m.add_argument("--model", choices=sorted(MODEL_SIZES), default="1b")
    m.add_argument("--hidden-size", type=int, default=None)
    m.add_argument("--num-layers", type=int, default=None)
    m.add_argument("--num-heads", type=int, default=None)
    m.add_argument("--num-kv-heads", type=int, default=None)
    m.add_argument("--intermediate-size", type=int, default=None)
    m.add_argument("--vocab-size", type=int, default=128256)
    m.add_argument("--tie-word-embeddings", action="store_true")
    t = p.add_argument_group("training")
    t.add_argument("--seed", type=int, default=42)
    t.add_argument("--steps", type=int, default=10000)
    t.add_argument("--mbs", type=int, default=2)
    t.add_argument("--acc", type=int, default=1)
    t.add_argument("--seq", type=int, default=4096)
    t.add_argument("--learning-rate", type=float, default=3e-4)
    t.add_argument("--min-lr", type=float, default=3e-5)
    t.add_argument("--weight-decay", type=float, default=0.01)
    t.add_argument("--grad-clip", type=float, default=1.0)
    t.add_argument("--warmup-steps", type=int, default=1000)
    par = p.add_argument_group("parallelism")
    par.add_argument("--dp", type=int, default=8)
    par.add_argument("--pp", type=int, default=1)
    par.add_argument("--tp", type=int, default=1)
    par.add_argument("--cp", type=int, default=1)
    par.add_argument("--ep", type=int, default=1)
    par.add_argument("--zero", type=int, default=1, choices=[0, 1])
    d = p.add_argument_group("data / io")
    d.add_argument("--dataset", type=str, default=None, help="folder of .ds token files; omitted: dummy data")
    d.add_argument("--tokenizer", type=str, default=None)
    d.add_argument("--checkpoints-path", type=str, default="checkpoints")
    d.add_argument("--save-interval", type=int, default=1000)
    d.add_argument("--configs-path", type=str, default="logs/configs")
    d.add_argument("--slurm-logs-path", type=str, default="logs/slurm_logs")
    d.add_argument("--slurm-scripts-dir", type=str, default="logs/slurm_scripts")
    d.add_argument("--profiler-export-path", type=str, default=None)
    d.add_argument("--bench", type=str, default=None, help="benchmark csv path (sets NANOTRON_BENCHMARK=1)")
    return p.parse_args()


def create_config(a) -> Config:
    preset = MODEL_SIZES[a.model]
    h, L, nh, nkv, inter = preset if preset is not None else (a.hidden_size, a.num_layers, a.num_heads, a.num_kv_heads, a.intermediate_size)
    h, L, nh, nkv, inter = a.hidden_size or h, a.num_layers or L, a.num_heads or nh, a.num_kv_heads or nkv, a.intermediate_size or inter
    assert None not in (h, L, nh, nkv, inter), "custom model needs --hidden-size --num-layers --num-heads --num-kv-heads --intermediate-size"
    assert a.dp * a.pp * a.tp * a.cp == a.nodes * a.gpus_per_node, f"dp*pp*tp*cp={a.dp * a.pp * a.tp * a.cp} != nodes*gpus_per_node={a.nodes * a.gpus_per_node}"
    model_config = Qwen2Config(hidden_size=h, num_hidden_layers=L, num_attention_heads=nh, num_key_value_heads=nkv, intermediate_size=inter, vocab_size=a.vocab_size, max_position_embeddings=a.seq, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=a.tie_word_embeddings)
    dataset = NanosetDatasetsArgs(dataset_folder=a.dataset) if a.dataset else None
    return Config(
        general=GeneralArgs(project="nanotron", run=a.run, seed=a.seed, ignore_sanity_checks=True, benchmark_csv_path=a.bench),
        checkpoints=CheckpointsArgs(checkpoints_path=os.path.join(a.checkpoints_path, a.run), checkpoint_interval=a.save_interval, save_initial_state=False),
        parallelism=ParallelismArgs(dp=a.dp, pp=a.pp, tp=a.tp, context_parallel_size=a.cp, expert_parallel_size=a.ep, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
        model=ModelArgs(model_config=model_config, init_method=RandomInit(std=0.02), dtype="bfloat16"),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=a.tokenizer),
        logging=LoggingArgs(log_level="info", log_level_replica="info", iteration_step_info_interval=1),
        tokens=TokensArgs(sequence_length=a.seq, train_steps=a.steps, micro_batch_size=a.mbs, batch_accumulation_per_replica=a.acc),
        optimizer=OptimizerArgs(
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True), zero_stage=a.zero,
            weight_decay=a.weight_decay, clip_grad=a.grad_clip, accumulate_grad_in_fp32=True,
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=a.learning_rate, lr_warmup_steps=min(a.warmup_steps, max(1, a.steps // 10)), lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=a.min_lr),
        ),
        data_stages=[DatasetStageArgs(name="Stable Training Stage", start_training_step=1, data=DataArgs(dataset=dataset, seed=a.seed, num_loading_workers=1))],
        profiler=ProfilerArgs(profiler_export_path=a.profiler_export_path) if a.profiler_export_path else None,
    )


def create_slurm_script(a, config_path: str) -> str:
    repo = os.path.dirname(os.path.abspath(__file__))
    os.makedirs(a.slurm_logs_path, exist_ok=True)
    lines = [
        "#!/bin/bash",
        f"#SBATCH --job-name={a.run}",
        f"#SBATCH --nodes={a.nodes}",
        "#SBATCH --ntasks-per-node=1",
        f"#SBATCH --gpus-per-node={a.gpus_per_node}",
        f"#SBATCH --partition={a.partition}",
        f"#SBATCH --qos={a.qos}",
        f"#SBATCH --time={a.time_limit}",
        f"#SBATCH --output={a.slurm_logs_path}/%x-%j.out",
        "#SBATCH --exclusive",
    ]
    if a.reservation:
        lines.append(f"#SBATCH --reservation={a.reservation}")
    lines += [
        "set -x -e",
        a.env or "",
        'export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)',
        "export MASTER_PORT=$((1024 + RANDOM % 64511))",
        "export CUDA_DEVICE_MAX_CONNECTIONS=1",
        "export NCCL_DEBUG=WARN",
    ]
    if a.bench:
        lines.append("export NANOTRON_BENCHMARK=1")
    lines += [
        f"cd {repo}",
        "srun -u bash -c \"torchrun --nnodes $SLURM_NNODES --nproc_per_node " + str(a.gpus_per_node) + " --node_rank \\$SLURM_PROCID --rdzv_backend c10d "
        "--rdzv_endpoint $MASTER_ADDR:$MASTER_PORT --max_restarts 0 --tee 3 run_train.py --config-file " + config_path + "\"",
    ]
    return "\n".join(l for l in lines if l != "") + "\n"


def main():
    a = parse_args()
    config = create_config(a)
    os.makedirs(a.configs_path, exist_ok=True)
    os.makedirs(a.slurm_scripts_dir, exist_ok=True)
    config_path = os.path.abspath(os.path.join(a.configs_path, f"{a.run}.yaml"))
    config.save_as_yaml(config_path)
    script_path = os.path.join(a.slurm_scripts_dir, f"{a.run}.slurm")
    with open(script_path, "w") as f:
        f.write(create_slurm_script(a, config_path))
    tokens = config.global_batch_size_in_tokens
    print(f"config: {config_path}\nscript: {script_path}\nglobal batch: {tokens} tokens, {a.steps} steps = {tokens * a.steps / 1e9:.2f}B tokens")
    if a.dry_run:
        return
    if shutil.which("sbatch") is None:
        raise SystemExit("sbatch not found; use --dry-run to only write the files")
    out = subprocess.run(["sbatch", script_path], capture_output=True, text=True)
    print(out.stdout.strip() or out.stderr.strip())
    if a.show_logs and out.returncode == 0:
        job_id = out.stdout.strip().split()[-1]
        log = os.path.join(a.slurm_logs_path, f"{a.run}-{job_id}.out")
        while not os.path.exists(log):
            time.sleep(1)
        subprocess.run(["tail", "-f", log])


if __name__ == "__main__":
    main()
