#!/usr/bin/env python
"""Builds a training config from command-line presets and submits it to slurm (parity: reference slurm_launcher.py).

    python slurm_launcher.py --run my_run --model 1b --nodes 2 --dp 16 --tp 1 --pp 1 --seq 4096 --mbs 2 --acc 8 --steps 1000 --dry-run

Writes ``<configs-path>/<run>.yaml`` and ``<slurm-scripts-dir>/<run>.slurm``; ``--dry-run`` stops there, otherwise the
script is handed to ``sbatch`` (``--chain N`` submits N jobs, each starting after the previous one ended).

Recovery is checkpoint + resubmit, not in-job restarts: torchrun runs with ``--max_restarts 0``; slurm sends SIGUSR1 to the
batch shell ``--signal-lead`` seconds before the time limit, the script creates the run's kill-switch file
(``NANOTRON_KILL_SWITCH``, which the trainer polls at every step boundary and agrees on across ranks), the trainer saves a
checkpoint and leaves, and the job requeues itself (``--requeue``) or the next job of the chain takes over.  Touching that
file by hand stops a run the same way.  Every start resumes from ``<checkpoints-path>/<run>/latest.txt`` when it exists.
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
    OptimizerArgs, ParallelismArgs, PretrainDatasetsArgs, ProfilerArgs, Qwen2Config, RandomInit, TokenizerArgs, TokensArgs,
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


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="nanotron_b200 slurm launcher")
    p.add_argument("--run", type=str, default="nanotron", help="run name")
    p.add_argument("--project", type=str, default="nanotron", help="project name for logging")
    g = p.add_argument_group("slurm")
    g.add_argument("--gpus-per-node", type=int, default=8)
    g.add_argument("--cpus-per-task", type=int, default=None, help="CPU cores of the one task per node (default: slurm's)")
    g.add_argument("--partition", type=str, default="b200")
    g.add_argument("--qos", type=str, default="normal")
    g.add_argument("--account", type=str, default=None)
    g.add_argument("--time-limit", type=str, default="24:00:00")
    g.add_argument("--nodes", type=int, default=None, help="default: dp*pp*tp*cp / gpus-per-node")
    g.add_argument("--reservation", type=str, default=None)
    g.add_argument("--nodelist", type=str, default=None)
    g.add_argument("--exclude", type=str, default=None)
    g.add_argument("--email", type=str, default=None, help="BEGIN / END / FAIL notifications")
    g.add_argument("--tmp-dir", type=str, default="/tmp", help="TMPDIR on the compute nodes")
    g.add_argument("--pre-launch-commands", type=str, default="", help="shell lines run on the batch node before srun (module loads, checks)")
    g.add_argument("--extra-env", type=str, default="", help="KEY=VALUE pairs, comma or blank separated, exported in the job")
    g.add_argument("--env", type=str, default=None, help="conda/venv activate line")
    g.add_argument("--requeue", action="store_true", help="let the job requeue itself after the pre-time-limit checkpoint")
    g.add_argument("--signal-lead", type=int, default=300, help="seconds before the time limit at which the clean stop is requested (0: no signal)")
    g.add_argument("--chain", type=int, default=1, help="submit this many jobs, each depending on the end of the previous one")
    g.add_argument("--dry-run", action="store_true")
    g.add_argument("--show-logs", action="store_true")
    m = p.add_argument_group("model")
    m.add_argument("--model", choices=sorted(MODEL_SIZES), default="1b")
    m.add_argument("--hidden-size", type=int, default=None)
    m.add_argument("--num-layers", type=int, default=None)
    m.add_argument("--num-heads", type=int, default=None)
    m.add_argument("--num-kv-heads", type=int, default=None)
    m.add_argument("--intermediate-size", type=int, default=None)
    m.add_argument("--vocab-size", type=int, default=128256)
    m.add_argument("--tie-word-embeddings", action="store_true")
    m.add_argument("--attention", type=str, default=None, help="_attn_implementation of the model config (default: the in-tree flash attention)")
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
    t.add_argument("--recompute-layer", action="store_true")
    par = p.add_argument_group("parallelism")
    par.add_argument("--dp", type=int, default=8)
    par.add_argument("--pp", type=int, default=1)
    par.add_argument("--tp", type=int, default=1)
    par.add_argument("--cp", type=int, default=1)
    par.add_argument("--ep", type=int, default=1)
    par.add_argument("--zero", type=int, default=1, choices=[0, 1])
    par.add_argument("--pp-engine", type=str, default="1f1b", choices=["1f1b", "afab"])
    d = p.add_argument_group("data / io")
    d.add_argument("--dataset", type=str, default=None, help="folder of .ds token files (nanoset), or with --text-column a Hugging Face dataset name / path; omitted: dummy data")
    d.add_argument("--text-column", type=str, default=None, help="treat --dataset as a Hugging Face text dataset and tokenize this column")
    d.add_argument("--tokenizer", type=str, default=None)
    d.add_argument("--num-loading-workers", type=int, default=1)
    d.add_argument("--checkpoints-path", type=str, default="checkpoints")
    d.add_argument("--save-interval", type=int, default=1000)
    d.add_argument("--save-initial-state", action="store_true")
    d.add_argument("--no-resume", action="store_true", help="start from scratch even when the run has a latest checkpoint")
    d.add_argument("--configs-path", type=str, default="logs/configs")
    d.add_argument("--slurm-logs-path", type=str, default="logs/slurm_logs")
    d.add_argument("--slurm-scripts-dir", type=str, default="logs/slurm_scripts")
    d.add_argument("--profiler-export-path", type=str, default=None)
    d.add_argument("--bench", type=str, default=None, help="benchmark csv path (sets NANOTRON_BENCHMARK=1)")
    lg = p.add_argument_group("logging")
    lg.add_argument("--enable-wandb", action="store_true", help="otherwise WANDB_MODE=disabled is exported")
    lg.add_argument("--log-lvl", type=str, default="info")
    lg.add_argument("--log-interval", type=int, default=1)
    lg.add_argument("--no-sanity", action="store_true", help="skip the runtime invariant checks")
    a = p.parse_args(argv)
    world = a.dp * a.pp * a.tp * a.cp
    if a.nodes is None:
        assert world % a.gpus_per_node == 0 or world < a.gpus_per_node, f"dp*pp*tp*cp={world} does not fill whole nodes of {a.gpus_per_node} GPUs"
        a.nodes = max(1, world // a.gpus_per_node)
        if world < a.gpus_per_node:
            a.gpus_per_node = world
    return a


def parse_extra_env(spec: str) -> dict:
    """"A=1,B=two C=3" -> {"A": "1", "B": "two", "C": "3"}."""
    out = {}
    for item in spec.replace(",", " ").split():
        assert "=" in item, f"--extra-env entries are KEY=VALUE, got {item!r}"
        k, v = item.split("=", 1)
        out[k] = v
    return out


def create_config(a) -> Config:
    preset = MODEL_SIZES[a.model]
    h, L, nh, nkv, inter = preset if preset is not None else (a.hidden_size, a.num_layers, a.num_heads, a.num_kv_heads, a.intermediate_size)
    h, L, nh, nkv, inter = a.hidden_size or h, a.num_layers or L, a.num_heads or nh, a.num_kv_heads or nkv, a.intermediate_size or inter
    assert None not in (h, L, nh, nkv, inter), "custom model needs --hidden-size --num-layers --num-heads --num-kv-heads --intermediate-size"
    assert a.dp * a.pp * a.tp * a.cp == a.nodes * a.gpus_per_node, f"dp*pp*tp*cp={a.dp * a.pp * a.tp * a.cp} != nodes*gpus_per_node={a.nodes * a.gpus_per_node}"
    assert nh % a.tp == 0 and nkv % a.tp == 0, f"tp={a.tp} must divide the {nh} query heads and the {nkv} key/value heads"
    assert L >= a.pp, f"{L} layers cannot fill {a.pp} pipeline stages"
    assert not (a.ep > 1 and a.zero), "expert parallelism is laid over the data-parallel ranks: use --zero 0 with --ep > 1"
    extra = {"_attn_implementation": a.attention} if a.attention else {}
    model_config = Qwen2Config(hidden_size=h, num_hidden_layers=L, num_attention_heads=nh, num_key_value_heads=nkv, intermediate_size=inter, vocab_size=a.vocab_size, max_position_embeddings=a.seq, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=a.tie_word_embeddings, **extra)
    if a.dataset and a.text_column:
        assert a.tokenizer, "a text dataset needs --tokenizer"
        dataset = PretrainDatasetsArgs(hf_dataset_or_datasets=a.dataset, text_column_name=a.text_column)
    elif a.dataset:
        dataset = NanosetDatasetsArgs(dataset_folder=a.dataset)
    else:
        dataset = None
    run_dir = os.path.join(a.checkpoints_path, a.run)
    resume = run_dir if (not a.no_resume and os.path.exists(os.path.join(run_dir, "latest.txt"))) else None
    return Config(
        general=GeneralArgs(project=a.project, run=a.run, seed=a.seed, ignore_sanity_checks=a.no_sanity, benchmark_csv_path=a.bench),
        checkpoints=CheckpointsArgs(checkpoints_path=run_dir, checkpoint_interval=a.save_interval, save_initial_state=a.save_initial_state, resume_checkpoint_path=resume),
        parallelism=ParallelismArgs(dp=a.dp, pp=a.pp, tp=a.tp, context_parallel_size=a.cp, expert_parallel_size=a.ep, pp_engine=a.pp_engine, tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True, recompute_layer=a.recompute_layer),
        model=ModelArgs(model_config=model_config, init_method=RandomInit(std=0.02), dtype="bfloat16"),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=a.tokenizer),
        logging=LoggingArgs(log_level=a.log_lvl, log_level_replica=a.log_lvl, iteration_step_info_interval=a.log_interval),
        tokens=TokensArgs(sequence_length=a.seq, train_steps=a.steps, micro_batch_size=a.mbs, batch_accumulation_per_replica=a.acc),
        optimizer=OptimizerArgs(
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True), zero_stage=a.zero,
            weight_decay=a.weight_decay, clip_grad=a.grad_clip, accumulate_grad_in_fp32=True,
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=a.learning_rate, lr_warmup_steps=min(a.warmup_steps, max(1, a.steps // 10)), lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=a.min_lr),
        ),
        data_stages=[DatasetStageArgs(name="Stable Training Stage", start_training_step=1, data=DataArgs(dataset=dataset, seed=a.seed, num_loading_workers=a.num_loading_workers))],
        profiler=ProfilerArgs(profiler_export_path=a.profiler_export_path) if a.profiler_export_path else None,
    )


def create_slurm_script(a, config_path: str) -> str:
    repo = os.path.dirname(os.path.abspath(__file__))
    os.makedirs(a.slurm_logs_path, exist_ok=True)
    run_dir = os.path.join(a.checkpoints_path, a.run)
    sb = [
        "#!/bin/bash",
        f"#SBATCH --job-name={a.run}",
        f"#SBATCH --nodes={a.nodes}",
        "#SBATCH --ntasks-per-node=1",  # one torchrun per node, which starts one rank per GPU
        f"#SBATCH --gpus-per-node={a.gpus_per_node}",
        f"#SBATCH --partition={a.partition}",
        f"#SBATCH --qos={a.qos}",
        f"#SBATCH --time={a.time_limit}",
        f"#SBATCH --output={a.slurm_logs_path}/%x-%j.out",
        "#SBATCH --exclusive",
        "#SBATCH --wait-all-nodes=1",
    ]
    for flag, value in (("cpus-per-task", a.cpus_per_task), ("account", a.account), ("reservation", a.reservation), ("nodelist", a.nodelist), ("exclude", a.exclude)):
        if value:
            sb.append(f"#SBATCH --{flag}={value}")
    if a.email:
        sb += ["#SBATCH --mail-type=BEGIN,END,FAIL", f"#SBATCH --mail-user={a.email}"]
    if a.signal_lead > 0:
        sb.append(f"#SBATCH --signal=B:USR1@{a.signal_lead}")  # to the batch shell only; the trap below passes it on
    if a.requeue:
        sb += ["#SBATCH --requeue", "#SBATCH --open-mode=append"]
    lines = sb + [
        "set -x -e",
        'echo "START TIME: $(date)  job $SLURM_JOB_ID on $SLURM_JOB_NODELIST"',
        a.env or "",
        *[l for l in a.pre_launch_commands.splitlines() if l.strip()],
        'export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)',
        "export MASTER_PORT=$((1024 + RANDOM % 64511))",
        f"export TMPDIR={a.tmp_dir}",
        "export CUDA_DEVICE_MAX_CONNECTIONS=1",
        "export NCCL_DEBUG=WARN",
        "export TORCH_NCCL_ASYNC_ERROR_HANDLING=1",
        f"export NANOTRON_KILL_SWITCH={os.path.abspath(run_dir)}/STOP",  # touch this file to stop the run at the next step boundary
        f"mkdir -p {os.path.abspath(run_dir)}",
        'rm -f "$NANOTRON_KILL_SWITCH"',  # a stop request belongs to the job that received it
    ]
    if not a.enable_wandb:
        lines.append("export WANDB_MODE=disabled")
    if a.bench:
        lines.append("export NANOTRON_BENCHMARK=1")
    lines += [f"export {k}={v}" for k, v in parse_extra_env(a.extra_env).items()]
    launcher = ("torchrun --nnodes $SLURM_NNODES --nproc_per_node " + str(a.gpus_per_node) + " --node_rank \\$SLURM_PROCID --rdzv_backend c10d "
                "--rdzv_endpoint $MASTER_ADDR:$MASTER_PORT --max_restarts 0 --tee 3 run_train.py --config-file " + config_path)
    lines += [f"cd {repo}"]
    if a.signal_lead > 0:
        lines += [
            "# the time limit is near: the kill-switch file makes every rank stop cleanly (checkpoint at the next step boundary)",
            "stop_requested=0",
            "trap 'stop_requested=1; touch \"$NANOTRON_KILL_SWITCH\"' USR1",
            f'srun -u bash -c "{launcher}" &',
            "srun_pid=$!",
            "set +e",
            "wait $srun_pid; rc=$?",
            'if [ "$stop_requested" = 1 ]; then wait $srun_pid; rc=$?; fi',  # the first wait returns when the trap fires
        ]
        if a.requeue:
            lines.append('if [ "$stop_requested" = 1 ] && [ -f ' + os.path.abspath(run_dir) + '/latest.txt ]; then scontrol requeue $SLURM_JOB_ID; fi')
        lines += ['echo "END TIME: $(date)  exit code $rc"', "exit $rc"]
    else:
        lines += [f'srun -u bash -c "{launcher}"', 'echo "END TIME: $(date)"']
    return "\n".join(l for l in lines if l != "") + "\n"


def submit(script_path: str, dependency: str = None, run=subprocess.run) -> str:
    """sbatch the script (after job `dependency` ended, if given); returns the job id."""
    cmd = ["sbatch"] + ([f"--dependency=afterany:{dependency}"] if dependency else []) + [script_path]
    out = run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise SystemExit(f"sbatch failed: {(out.stderr or out.stdout).strip()}")
    return out.stdout.strip().split()[-1]


def main(argv=None):
    a = parse_args(argv)
    config = create_config(a)
    os.makedirs(a.configs_path, exist_ok=True)
    os.makedirs(a.slurm_scripts_dir, exist_ok=True)
    config_path = os.path.abspath(os.path.join(a.configs_path, f"{a.run}.yaml"))
    config.save_as_yaml(config_path)
    script_path = os.path.join(a.slurm_scripts_dir, f"{a.run}.slurm")
    with open(script_path, "w") as f:
        f.write(create_slurm_script(a, config_path))
    tokens = config.global_batch_size_in_tokens
    print(f"config: {config_path}\nscript: {script_path}\nglobal batch: {tokens} tokens, {a.steps} steps = {tokens * a.steps / 1e9:.2f}B tokens on {a.nodes} node(s) x {a.gpus_per_node} GPUs")
    if config.checkpoints.resume_checkpoint_path is not None:
        print(f"resumes from {config.checkpoints.resume_checkpoint_path}")
    if a.dry_run:
        return
    if shutil.which("sbatch") is None:
        raise SystemExit("sbatch not found; use --dry-run to only write the files")
    job_id = None
    first = None
    for _ in range(max(1, a.chain)):
        job_id = submit(script_path, dependency=job_id)
        first = first or job_id
        print(f"submitted job {job_id}")
    if a.show_logs:
        log = os.path.join(a.slurm_logs_path, f"{a.run}-{first}.out")
        while not os.path.exists(log):
            time.sleep(1)
        subprocess.run(["tail", "-f", log])


if __name__ == "__main__":
    main()
