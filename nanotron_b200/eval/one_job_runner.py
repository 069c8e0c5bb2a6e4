"""Launches one evaluation job per uploaded checkpoint (parity: reference src/nanotron/eval/one_job_runner.py).

The runner is the ``post_upload_callback`` of the S3 mover: when a checkpoint finished uploading, it renders an sbatch
script that downloads the checkpoint, runs ``run_evals.py`` (lighteval) on it and uploads the results, then submits
it with ``sbatch``.  Without slurm on the machine (``sbatch`` missing) the script is still written, and the submission
step is reported as skipped, which is what the tests exercise.
"""
from __future__ import annotations

import datetime
import os
import re
import shutil
import subprocess
from typing import List, Optional, Tuple

from nanotron_b200 import logging
from nanotron_b200.config import Config, LightEvalConfig
from nanotron_b200.logging import log_rank
from nanotron_b200.parallel import ParallelContext

logger = logging.get_logger(__name__)


class LightEvalRunner:
    def __init__(self, config: Config, parallel_context: Optional[ParallelContext] = None):
        self.config = config
        assert config.lighteval is not None, "LightEval config is required"
        self.lighteval_config: LightEvalConfig = config.lighteval
        self.parallel_context = parallel_context

    def eval_single_checkpoint(self, uploaded_files: str) -> Tuple[Optional[str], Optional[str]]:
        """``uploaded_files``: the s5cmd json log of the upload.  Returns (slurm job id, slurm log path)."""
        checkpoint_path = self._checkpoint_from_upload_log(uploaded_files)
        if checkpoint_path is None:
            log_rank("No model checkpoint found in the upload log: evaluation not launched", logger=logger, level=logging.WARNING)
            return None, None
        step = self._step_from_path(checkpoint_path)
        if self.lighteval_config.eval_interval and step is not None and step % self.lighteval_config.eval_interval != 0:
            return None, None
        script_path, log_path = self.render_slurm_script(checkpoint_path, step)
        job_id = self.submit(script_path)
        return job_id, log_path

    @staticmethod
    def _checkpoint_from_upload_log(uploaded_files: str) -> Optional[str]:
        for line in uploaded_files.splitlines():
            m = re.search(r"(s3://[^\s\"']+?/\d+)/(config\.yaml|model/)", line)
            if m:
                return m.group(1)
        return None

    @staticmethod
    def _step_from_path(path: str) -> Optional[int]:
        m = re.search(r"/(\d+)/?$", path)
        return int(m.group(1)) if m else None

    def render_slurm_script(self, checkpoint_s3_path: str, step: Optional[int]) -> Tuple[str, str]:
        le = self.lighteval_config
        slurm = le.slurm
        run = self.config.general.run
        stamp = datetime.datetime.now().strftime("%Y%m%d_%H%M%S")
        script_dir = str(le.slurm_script_dir)
        logs_dir = str(le.logs_path)
        os.makedirs(script_dir, exist_ok=True)
        os.makedirs(logs_dir, exist_ok=True)
        name = f"eval_{run}_{step}_{stamp}"
        log_path = os.path.join(logs_dir, f"{name}.out")
        local_ckpt = os.path.join(str(le.local_checkpoint_dir), run, str(step))
        par = le.parallelism
        n_gpus = par.dp * par.pp * par.tp
        nodes = max(1, (n_gpus + slurm.gpus_per_node - 1) // slurm.gpus_per_node)
        lines = [
            "#!/bin/bash",
            f"#SBATCH --job-name={name}",
            f"#SBATCH --partition={slurm.partition}",
            f"#SBATCH --nodes={nodes}",
            f"#SBATCH --gpus-per-node={min(n_gpus, slurm.gpus_per_node)}",
            f"#SBATCH --cpus-per-task={slurm.cpus_per_task}",
            f"#SBATCH --qos={slurm.qos}",
            f"#SBATCH --time={slurm.time}",
            f"#SBATCH --output={log_path}",
        ]
        if slurm.reservation:
            lines.append(f"#SBATCH --reservation={slurm.reservation}")
        lines += [
            "set -e",
            f"export HF_HOME={slurm.hf_cache}",
            "export CUDA_DEVICE_MAX_CONNECTIONS=1",
            f"mkdir -p {local_ckpt}",
            f"s5cmd cp --exclude 'optimizer/*' --exclude 'random/*' --exclude 'lr_scheduler/*' '{checkpoint_s3_path}/*' {local_ckpt}/",
            f"cd {le.nanotron_path or '.'}",
            f"torchrun --nproc_per_node {min(n_gpus, slurm.gpus_per_node)} --nnodes {nodes} --master-addr 127.0.0.1 run_evals.py "
            f"--checkpoint-config-path {local_ckpt}/config.yaml" + (f" --lighteval-override {le.eval_config_override}" if le.eval_config_override else ""),
        ]
        if le.s3_save_path:
            lines.append(f"s5cmd cp '{le.output_dir or 'eval_results'}/*' {le.s3_save_path}/{run}/{step}/")
        if le.upload_to_wandb and le.wandb_project:
            lines.append(f"python -m nanotron_b200.eval.upload_to_wandb --wandb_project {le.wandb_project} --wandb_entity {le.wandb_entity or ''} --model_name {run} --results_path {le.output_dir or 'eval_results'} --train_step {step}")
        script_path = os.path.join(script_dir, f"{name}.slurm")
        with open(script_path, "w") as f:
            f.write("\n".join(lines) + "\n")
        return script_path, log_path

    @staticmethod
    def submit(script_path: str) -> Optional[str]:
        if shutil.which("sbatch") is None:
            log_rank(f"sbatch not found: evaluation script written to {script_path} but not submitted", logger=logger, level=logging.WARNING)
            return None
        res = subprocess.run(["sbatch", script_path], capture_output=True, text=True)
        if res.returncode != 0:
            log_rank(f"sbatch failed ({res.returncode}): {res.stderr.strip()}", logger=logger, level=logging.ERROR)
            return None
        m = re.search(r"(\d+)", res.stdout)
        return m.group(1) if m else None
