"""Evaluation-job section of the config (parity: reference src/nanotron/config/lighteval_config.py)."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional, Union

from nanotron_b200.config.parallelism_config import ParallelismArgs
from nanotron_b200.config.utils_config import SamplerType

DEFAULT_SEED = 42


@dataclass
class GenerationArgs:
    sampler: Optional[Union[str, SamplerType]] = None
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
        if self.seed is None:
            self.seed = DEFAULT_SEED


@dataclass
class LightEvalLoggingArgs:
    output_dir: Optional[str] = None
    save_details: bool = True
    push_to_hub: bool = False
    push_to_tensorboard: bool = False
    public_run: bool = False
    results_org: Optional[str] = None
    tensorboard_metric_prefix: str = "eval"

    def __post_init__(self):
        if isinstance(self.output_dir, Path):
            self.output_dir = str(self.output_dir)


@dataclass
class LightEvalTasksArgs:
    tasks: Union[str, list] = "early-signal"
    custom_tasks: Optional[str] = None
    max_samples: Optional[int] = None
    num_fewshot_seeds: Optional[int] = None
    dataset_loading_processes: int = 8
    multichoice_continuations_start_space: Optional[bool] = None


@dataclass
class LightEvalWandbLoggerConfig:
    wandb_project: str = ""
    wandb_entity: Optional[str] = None
    wandb_run_name: Optional[str] = None

    def __post_init__(self):
        assert self.wandb_project != "", "Please specify a wandb_project"


@dataclass
class LightEvalSlurm:
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
    """Settings for the evaluation job started after a checkpoint upload."""

    slurm_script_dir: Optional[Path] = Path("eval_results/launch-config")
    logs_path: Optional[Path] = Path("eval_results/logs")
    local_checkpoint_dir: Path = Path("/scratch")
    parallelism: Optional[ParallelismArgs] = None
    batch_size: Optional[int] = None
    generation: Optional[Union[GenerationArgs, Dict[str, GenerationArgs]]] = None
    tasks: Optional[LightEvalTasksArgs] = None
    logging: Optional[LightEvalLoggingArgs] = None
    wandb: Optional[LightEvalWandbLoggerConfig] = None
    slurm: Optional[LightEvalSlurm] = None
    s3_save_path: Optional[str] = None
    upload_to_wandb: Optional[bool] = False
    wandb_project: Optional[str] = None
    wandb_entity: Optional[str] = None
    output_dir: Optional[str] = None
    nanotron_path: Optional[str] = "./"
    eval_config_override: Optional[str] = None
    eval_interval: Optional[int] = None
    eval_interval_file: Optional[Path] = None

    def __post_init__(self):
        if self.parallelism is None:
            self.parallelism = ParallelismArgs(dp=1, pp=1, tp=1)
        if self.slurm is None:
            self.slurm = LightEvalSlurm()
        if self.tasks is None:
            self.tasks = LightEvalTasksArgs()
