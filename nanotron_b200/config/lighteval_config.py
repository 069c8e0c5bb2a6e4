"""Evaluation section of the config: how text is sampled (``GenerationArgs``) and how the evaluation job that follows a
checkpoint upload is set up (``LightEvalConfig`` and its sub-sections).
Schema parity: reference src/nanotron/config/lighteval_config.py; every key of that schema loads, keys of newer lighteval
releases that mean the same are accepted beside them.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional, Union

from nanotron_b200.config.parallelism_config import ParallelismArgs
from nanotron_b200.config.utils_config import SamplerType

DEFAULT_SEED = 42  # of generation, and of the training sections that import it


@dataclass
class GenerationArgs:
    sampler: Optional[Union[str, SamplerType]] = None  # greedy / top_k / top_p / basic
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    n_samples: Optional[int] = None
    eos: Optional[str] = None
    seed: Optional[int] = None
    use_cache: Optional[bool] = False

    def __post_init__(self):
        if isinstance(self.sampler, str):
            self.sampler = SamplerType[self.sampler.upper()]
        self.seed = DEFAULT_SEED if self.seed is None else self.seed


@dataclass
class LightEvalLoggingArgs:
    """Where results go."""

    # the reference's keys
    local_output_path: Optional[Path] = None
    push_results_to_hub: Optional[bool] = None
    push_details_to_hub: Optional[bool] = None
    push_results_to_tensorboard: Optional[bool] = None
    hub_repo_results: Optional[str] = None
    hub_repo_details: Optional[str] = None
    hub_repo_tensorboard: Optional[str] = None
    tensorboard_metric_prefix: Optional[str] = None
    # spellings of newer lighteval releases
    output_dir: Optional[str] = None
    save_details: Optional[bool] = None
    push_to_hub: Optional[bool] = None
    push_to_tensorboard: Optional[bool] = None
    public_run: Optional[bool] = None
    results_org: Optional[str] = None

    def __post_init__(self):
        if self.local_output_path is None and self.output_dir is not None:
            self.local_output_path = self.output_dir
        if self.local_output_path is not None:
            self.local_output_path = Path(self.local_output_path)
            self.output_dir = str(self.local_output_path)
        if self.push_results_to_hub is None and self.push_to_hub is not None:
            self.push_results_to_hub = self.push_to_hub
        if self.push_results_to_tensorboard is None and self.push_to_tensorboard is not None:
            self.push_results_to_tensorboard = self.push_to_tensorboard


@dataclass
class LightEvalTasksArgs:
    """What is evaluated: a task group or a comma-separated list (``nanotron_b200/eval/evaluation_tasks.py`` has the names)."""

    tasks: Optional[Union[str, list]] = None
    custom_tasks: Optional[str] = None
    max_samples: Optional[int] = None
    num_fewshot_seeds: Optional[int] = None
    dataset_loading_processes: Optional[int] = 8
    multichoice_continuations_start_space: Optional[bool] = None
    no_multichoice_continuations_start_space: Optional[bool] = None

    def __post_init__(self):
        if self.tasks is None:
            self.tasks = "early-signal"
        if self.multichoice_continuations_start_space and self.no_multichoice_continuations_start_space:
            raise ValueError("multichoice_continuations_start_space and no_multichoice_continuations_start_space exclude each other")


@dataclass
class LightEvalWandbLoggerConfig:
    wandb_project: str = ""
    wandb_entity: Optional[str] = None
    wandb_run_name: Optional[str] = None

    def __post_init__(self):
        if not self.wandb_project:
            raise AssertionError("Please specify a wandb_project")


@dataclass
class LightEvalSlurm:
    """Resources of the evaluation job."""

    gpus_per_node: int = 8
    partition: str = "hopper-prod"
    hf_cache: str = "~/.cache/huggingface"
    cpus_per_task: int = 88
    qos: str = "low"
    time: str = "24:00:00"
    reservation: Optional[str] = "smollm"

    def __post_init__(self):
        self.hf_cache = str(Path(self.hf_cache).expanduser())


@dataclass
class LightEvalConfig:
    """The evaluation job started after a checkpoint upload.  Everything is optional: the same class overrides a saved
    configuration when an evaluation is launched by hand."""

    slurm_script_dir: Optional[Path] = Path("eval_results/launch-config")
    logs_path: Optional[Path] = Path("eval_results/logs")
    local_checkpoint_dir: Path = Path("/scratch")  # checkpoints are fetched to <local_checkpoint_dir>/<run>/<step>
    parallelism: Optional[ParallelismArgs] = None
    batch_size: Optional[int] = None
    generation: Optional[Union[GenerationArgs, Dict[str, GenerationArgs]]] = None
    tasks: Optional[LightEvalTasksArgs] = None
    logging: Optional[LightEvalLoggingArgs] = None
    wandb: Optional[LightEvalWandbLoggerConfig] = None
    slurm: Optional[LightEvalSlurm] = None
    s3_save_path: Optional[str] = None  # results are copied to <s3_save_path>/<run>/<step>/
    upload_to_wandb: Optional[bool] = False
    wandb_project: Optional[str] = None
    wandb_entity: Optional[str] = None
    output_dir: Optional[str] = None
    nanotron_path: Optional[str] = "./"
    eval_config_override: Optional[Union[str, Path]] = None
    eval_interval: Optional[int] = None  # a multiple of checkpoint_interval; None: after every uploaded checkpoint
    eval_interval_file: Optional[Path] = None  # when given, the interval is re-read from this file before every evaluation

    def __post_init__(self):
        self.parallelism = self.parallelism or ParallelismArgs(dp=1, pp=1, tp=1)
        self.slurm = self.slurm or LightEvalSlurm()
        self.tasks = self.tasks or LightEvalTasksArgs()
        self.local_checkpoint_dir = Path(self.local_checkpoint_dir).expanduser()
        if self.output_dir is None and self.logging is not None and self.logging.output_dir is not None:
            self.output_dir = self.logging.output_dir
        if self.upload_to_wandb:
            # (the entity may stay unset: wandb then uses the account's default)
            missing = [name for name in ("s3_save_path", "wandb_project") if getattr(self, name) is None]
            if missing:
                raise AssertionError(f"lighteval.upload_to_wandb needs {', '.join(missing)}")
        if self.eval_interval_file is not None and Path(self.eval_interval_file).exists():
            warnings.warn(f"{self.eval_interval_file} exists: `eval_interval` will be replaced by its content at the next evaluation")
