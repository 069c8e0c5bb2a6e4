"""Top-level ``Config`` and its sections; YAML round trip (parity: reference src/nanotron/config/config.py).

Section and field names equal the reference's so existing YAML files load unchanged.  Additions are optional
fields with defaults (e.g. ``OptimizerArgs.fused_zero_comm``, ``KernelArgs``).
"""
from __future__ import annotations

import datetime
import glob
import os
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import List, Optional, Type, Union

import torch
import yaml
from yaml.loader import SafeLoader

from nanotron_b200.config.lighteval_config import DEFAULT_SEED, GenerationArgs, LightEvalConfig
from nanotron_b200.config.models_config import (
    ExistingCheckpointInit,
    LlamaConfig,
    NanotronConfigs,
    Qwen2Config,
    RandomInit,
    SpectralMupInit,
    Starcoder2Config,
)
from nanotron_b200.config.parallelism_config import ParallelismArgs
from nanotron_b200.config.utils_config import (
    ConfigError,
    cast_str_to_torch_dtype,
    from_dict,
    serialize,
)
from nanotron_b200.logging import get_logger, human_format

logger = get_logger(__name__)
_LEVELS = ["debug", "info", "warning", "error", "critical", "passive"]


@dataclass
class BenchArgs:
    model_name: str
    sequence_length: int
    micro_batch_size: int
    batch_accumulation_per_replica: int
    benchmark_csv_path: str


@dataclass
class LoggingArgs:
    log_level: Optional[str] = None
    log_level_replica: Optional[str] = None
    iteration_step_info_interval: Optional[int] = 1

    def __post_init__(self):
        if self.log_level is None:
            self.log_level = "info"
        if self.log_level not in _LEVELS:
            raise ValueError(f"log_level should be a string selected in {_LEVELS} and not {self.log_level}")
        if self.log_level_replica is None:
            self.log_level_replica = "info"
        if self.log_level_replica not in _LEVELS:
            raise ValueError(f"log_level_replica should be a string selected in {_LEVELS} and not {self.log_level_replica}")


@dataclass
class MetricsLoggingArgs:
    log_level: int = 0
    log_detail_interval: int = 10

    def __post_init__(self):
        if self.log_level not in [0, 1]:
            raise ValueError(f"metrics log_level should be either 0 (basic) or 1 (full) and not {self.log_level}")
        if self.log_detail_interval <= 0:
            raise ValueError(f"log_detail_interval should be a positive integer and not {self.log_detail_interval}")


@dataclass
class PretrainDatasetsArgs:
    hf_dataset_or_datasets: Union[str, list, dict]
    hf_dataset_splits: Optional[Union[str, list]] = None
    hf_dataset_config_name: Optional[str] = None
    dataset_processing_num_proc_per_process: Optional[int] = 1
    dataset_overwrite_cache: Optional[bool] = False
    text_column_name: Optional[str] = None

    def __post_init__(self):
        if self.text_column_name is None:
            self.text_column_name = "text"
        if self.hf_dataset_splits is None:
            self.hf_dataset_splits = "train"


@dataclass
class SFTDatasetsArgs:
    hf_dataset_or_datasets: Union[str, list, dict]
    hf_dataset_splits: Optional[Union[str, list]] = None
    hf_dataset_config_name: Optional[str] = None
    dataset_processing_num_proc_per_process: Optional[int] = 1
    dataset_overwrite_cache: Optional[bool] = False
    sft_dataloader: Optional[bool] = True
    debug_max_samples: Optional[int] = None

    def __post_init__(self):
        if self.hf_dataset_splits is None:
            self.hf_dataset_splits = "train"


@dataclass
class S3UploadArgs:
    upload_s3_path: Path
    remove_after_upload: bool
    s5cmd_numworkers: Optional[int]
    s5cmd_concurrency: Optional[int]
    s5cmd_path: Optional[Path]

    def __post_init__(self):
        if isinstance(self.upload_s3_path, Path):
            # pathlib collapses "s3://" to "s3:/"; keep remote URLs as strings
            s = str(self.upload_s3_path)
            self.upload_s3_path = s.replace("s3:/", "s3://", 1) if s.startswith("s3:/") and not s.startswith("s3://") else s
        if isinstance(self.s5cmd_path, str):
            self.s5cmd_path = Path(self.s5cmd_path)


@dataclass
class NanosetDatasetsArgs:
    dataset_folder: Union[str, List[str]]
    dataset_weights: Optional[List[float]] = None
    dataset_read_path: Optional[Union[str, List[str]]] = None
    tokenizer_name: Optional[str] = None
    vocab_size: Optional[int] = None
    token_size_in_bytes: Optional[int] = None
    return_positions: Optional[bool] = True
    skip_in_stream: Optional[bool] = False
    pad_samples_to_global_batch_size: Optional[bool] = False
    dataset_max_tokens: Optional[List[int]] = None
    shuffle_files: Optional[bool] = False
    use_old_brrr_dataloader: Optional[bool] = False

    def __post_init__(self):
        if isinstance(self.dataset_folder, str):
            self.dataset_folder = [self.dataset_folder]
            self.dataset_weights = [1]
        if self.dataset_weights is not None and len(self.dataset_weights) != len(self.dataset_folder):
            raise ValueError(f"Number of dataset weights ({len(self.dataset_weights)}) does not match number of dataset folders ({len(self.dataset_folder)})")
        for folder in self.dataset_folder:
            metadata_files = glob.glob(os.path.join(folder, "*.metadata"))
            if not metadata_files:
                continue
            with open(metadata_files[0]) as f:
                first_line = f.readline().strip()
            if "|" in first_line:
                tokenizer_name, token_size = first_line.split("|")[:2]
                if self.tokenizer_name is None:
                    self.tokenizer_name = tokenizer_name
                    self.token_size_in_bytes = int(token_size)
                else:
                    assert self.tokenizer_name == tokenizer_name, f"Tokenizer name mismatch in datasets metadata: {self.tokenizer_name} vs {tokenizer_name}"
                    if self.token_size_in_bytes is not None:
                        assert self.token_size_in_bytes == int(token_size)
        if self.dataset_read_path is not None and not isinstance(self.dataset_read_path, str) and len(self.dataset_read_path) != len(self.dataset_folder):
            raise ValueError("Number of dataset read paths does not match number of dataset folders")


@dataclass
class DataArgs:
    dataset: Optional[Union[PretrainDatasetsArgs, NanosetDatasetsArgs, SFTDatasetsArgs]]  # None -> dummy generator
    seed: Optional[int]
    num_loading_workers: Optional[int] = 1

    def __post_init__(self):
        if self.seed is None:
            self.seed = DEFAULT_SEED


@dataclass
class DatasetStageArgs:
    name: str
    start_training_step: int
    data: DataArgs
    sequence_length: Optional[int] = None

    def __post_init__(self):
        if self.start_training_step < 0:
            raise ValueError(f"training_steps should be a positive integer and not {self.start_training_step}")


@dataclass
class CheckpointsArgs:
    checkpoints_path: Path
    checkpoint_interval: int
    save_initial_state: Optional[bool] = False
    save_final_state: Optional[bool] = True
    resume_checkpoint_path: Optional[Path] = None
    load_lr_scheduler: Optional[bool] = True
    load_optimizer: Optional[bool] = True
    checkpoints_path_is_shared_file_system: Optional[bool] = False

    def __post_init__(self):
        if isinstance(self.checkpoints_path, str):
            self.checkpoints_path = Path(self.checkpoints_path)
        if isinstance(self.resume_checkpoint_path, str):
            self.resume_checkpoint_path = Path(self.resume_checkpoint_path)


@dataclass
class GeneralArgs:
    project: str
    run: Optional[str] = None
    seed: Optional[int] = None
    step: Optional[int] = None
    consumed_train_samples: Optional[int] = None
    benchmark_csv_path: Optional[Path] = None
    ignore_sanity_checks: bool = True

    def __post_init__(self):
        if self.seed is None:
            self.seed = DEFAULT_SEED
        if self.run is None:
            self.run = "%date_%jobid"
        self.run = self.run.replace("%date", datetime.datetime.now().strftime("%Y%m%d_%H%M%S"))
        self.run = self.run.replace("%jobid", os.environ.get("SLURM_JOB_ID", "local"))


@dataclass
class ProfilerArgs:
    profiler_export_path: Optional[Path]
    wait: int = 1
    warmup: int = 1
    active: int = 1
    repeat: int = 1
    skip_first: int = 3
    record_shapes: bool = False
    profile_memory: bool = False
    with_stack: bool = True
    export_chrome_trace: bool = False


@dataclass
class KernelArgs:
    """Which implementation each hot op uses.  "auto": in-tree sm_100a kernels on CUDA, PyTorch math on CPU.
    "torch": always the PyTorch oracle.  ``gemm``: "cublas" routes plain GEMMs to the library, "tcgen05" to the
    in-tree kernel.  ``attention``: "auto" / "native" run the in-tree flash-attention kernels, "sdpa" the library kernel."""

    ops: str = "auto"
    gemm: str = "auto"
    attention: str = "auto"
    # operand precision of the linear-layer products: "bf16", or "fp8" = block-scaled fp8 (1 x 128 / 128 x 128 blocks, e4m3
    # forward, e5m2 gradients) for every tensor-parallel linear whose dimensions are multiples of 128
    linear: str = "bf16"


@dataclass
class ModelArgs:
    model_config: NanotronConfigs
    init_method: Union[RandomInit, SpectralMupInit, ExistingCheckpointInit]
    dtype: Optional[torch.dtype] = None
    make_vocab_size_divisible_by: int = 1
    ddp_bucket_cap_mb: int = 25

    def __post_init__(self):
        if self.dtype is None:
            self.dtype = torch.bfloat16
        if isinstance(self.dtype, str):
            self.dtype = cast_str_to_torch_dtype(self.dtype)
        if isinstance(self.model_config, dict):
            self.model_config = model_config_from_dict(self.model_config)
        self.model_config._is_using_mup = isinstance(self.init_method, SpectralMupInit)


@dataclass
class TokenizerArgs:
    tokenizer_name_or_path: Optional[str] = None
    tokenizer_revision: Optional[str] = None
    tokenizer_max_length: Optional[int] = None


@dataclass
class TokensArgs:
    sequence_length: int
    train_steps: int
    micro_batch_size: int
    batch_accumulation_per_replica: int
    val_check_interval: Optional[int] = -1
    limit_val_batches: Optional[int] = 0
    limit_test_batches: Optional[int] = 0


@dataclass
class LRSchedulerArgs:
    """lr_warmup_style: linear|constant; lr_decay_style: linear|cosine|1-sqrt; min_decay_lr defaults to learning_rate."""

    learning_rate: float
    lr_warmup_steps: int = 0
    lr_warmup_style: Optional[str] = None
    lr_decay_style: Optional[str] = None
    lr_decay_steps: Optional[int] = None
    lr_decay_starting_step: Optional[int] = None
    min_decay_lr: Optional[float] = None

    def __post_init__(self):
        if self.lr_warmup_style is None:
            self.lr_warmup_style = "linear"
        if self.lr_warmup_style not in ["linear", "constant"]:
            raise ValueError(f"lr_warmup_style should be a string selected in ['linear', 'constant'] and not {self.lr_warmup_style}")
        if self.lr_decay_style is None:
            self.lr_decay_style = "linear"
        if self.lr_decay_style not in ["linear", "cosine", "1-sqrt"]:
            raise ValueError(f"lr_decay_style should be a string selected in ['linear', 'cosine', '1-sqrt'] and not {self.lr_decay_style}")
        if self.min_decay_lr is None:
            self.min_decay_lr = self.learning_rate


@dataclass
class SGDOptimizerArgs:
    name: str = "sgd"


@dataclass
class AdamWOptimizerArgs:
    adam_eps: float
    adam_beta1: float
    adam_beta2: float
    torch_adam_is_fused: bool
    name: str = "adamW"


@dataclass
class OptimizerArgs:
    optimizer_factory: Union[SGDOptimizerArgs, AdamWOptimizerArgs]
    zero_stage: int
    weight_decay: float
    clip_grad: Optional[float]
    accumulate_grad_in_fp32: bool
    learning_rate_scheduler: LRSchedulerArgs
    weight_decay_exclude_named_params: Optional[List[str]] = None
    # None: use the in-kernel NVLink reduce-scatter + AdamW + all-gather step whenever it applies (CUDA, dp > 1 inside one
    # node, fp32 accumulation, AdamW).  False: always the NCCL collectives.
    fused_zero_comm: Optional[bool] = None
    # with the fused data-parallel step: start the gradient reduce-scatter of a layer while the last micro-batch's backward is still
    # running on the layers below it
    overlap_grad_reduce: bool = True

    def __post_init__(self):
        if self.weight_decay_exclude_named_params is None:
            self.weight_decay_exclude_named_params = []


@dataclass
class Config:
    general: GeneralArgs
    parallelism: ParallelismArgs
    model: ModelArgs
    tokenizer: Optional[TokenizerArgs] = None
    checkpoints: Optional[CheckpointsArgs] = None
    logging: Optional[LoggingArgs] = None
    metrics_logging: Optional[MetricsLoggingArgs] = None
    tokens: Optional[TokensArgs] = None
    optimizer: Optional[OptimizerArgs] = None
    data_stages: Optional[List[DatasetStageArgs]] = None
    profiler: Optional[ProfilerArgs] = None
    lighteval: Optional[LightEvalConfig] = None
    s3_upload: Optional[S3UploadArgs] = None
    kernels: Optional[KernelArgs] = None

    @classmethod
    def create_empty(cls):
        return cls(**{f.name: None for f in fields(cls)})

    def __post_init__(self):
        if self.s3_upload is not None and self.lighteval is not None and self.checkpoints is not None:
            if self.lighteval.eval_interval is None:
                self.lighteval.eval_interval = self.checkpoints.checkpoint_interval
            elif self.lighteval.eval_interval % self.checkpoints.checkpoint_interval != 0:
                raise ValueError(
                    f"eval_interval={self.lighteval.eval_interval} must be a multiple of checkpoint_interval={self.checkpoints.checkpoint_interval}"
                )
        if self.profiler is not None and self.profiler.profiler_export_path is not None and self.tokens is not None:
            p = self.profiler
            total = p.skip_first + p.repeat * (p.wait + p.warmup + p.active)
            assert self.tokens.train_steps >= total, f"Profiling needs train_steps >= skip_first + repeat*(wait+warmup+active) = {total}, got {self.tokens.train_steps}"
        if self.optimizer is not None and self.tokens is not None:
            sched = self.optimizer.learning_rate_scheduler
            if sched.lr_decay_steps is None:
                sched.lr_decay_steps = self.tokens.train_steps - sched.lr_warmup_steps
        if self.data_stages is not None:
            self.data_stages = sorted(self.data_stages, key=lambda s: s.start_training_step)
            names = [s.name for s in self.data_stages]
            steps = [s.start_training_step for s in self.data_stages]
            if not any(s == 1 for s in steps):
                raise ValueError("You must have a training stage starting at 1 in the config's data_stages")
            for s in self.data_stages:
                if names.count(s.name) > 1:
                    raise ValueError(f"Each stage should have unique names and not {names}")
                if steps.count(s.start_training_step) > 1:
                    raise ValueError(f"Each stage should have unique starting training step, please change the starting training step for stage {s.name}")
                if s.sequence_length is None and self.tokens is not None:
                    s.sequence_length = self.tokens.sequence_length
                if isinstance(s.data.dataset, NanosetDatasetsArgs) and s.data.dataset.vocab_size is not None and self.model is not None:
                    mv = self.model.model_config.vocab_size
                    if mv < s.data.dataset.vocab_size:
                        raise ValueError(f"Model vocab size ({mv}) is smaller than the dataset tokenizer's ({s.data.dataset.vocab_size})")
        if self.model is not None and self.parallelism is not None:
            mc = self.model.model_config
            tp = self.parallelism.tp
            nh = getattr(mc, "num_attention_heads", None)
            nkv = getattr(mc, "num_key_value_heads", None)
            if nh is not None:
                assert nh % tp == 0, f"num_attention_heads ({nh}) must be divisible by tp ({tp})"
            if nkv is not None and nh is not None:
                assert nkv >= tp or nkv == 1, f"num_key_value_heads ({nkv}) must be >= tp ({tp})"
                assert nh % nkv == 0, "num_attention_heads must be divisible by num_key_value_heads"

    @property
    def global_batch_size(self) -> int:
        return self.tokens.micro_batch_size * self.tokens.batch_accumulation_per_replica * self.parallelism.dp

    @property
    def global_batch_size_in_tokens(self) -> int:
        return self.global_batch_size * self.tokens.sequence_length

    def save_as_yaml(self, file_path: str, sanity_checks: bool = True):
        config_dict = serialize(self)
        file_path = str(file_path)
        os.makedirs(os.path.dirname(os.path.abspath(file_path)), exist_ok=True)
        with open(file_path, "w") as f:
            yaml.dump(config_dict, f, sort_keys=False)
        if sanity_checks:
            # re-parse what was written: a config that cannot be read back is a bug
            custom = type(self.model.model_config) if self.model is not None and type(self.model.model_config) not in (LlamaConfig, Qwen2Config, Starcoder2Config) else None
            get_config_from_file(file_path, config_class=self.__class__, model_config_class=custom)

    def get_yaml(self) -> str:
        return yaml.dump(serialize(self), sort_keys=False)

    @classmethod
    def load_from_yaml(cls, file_path: str):
        return get_config_from_file(file_path, config_class=cls)

    def as_dict(self) -> dict:
        return serialize(self)

    def print_config_details(self):
        mc = self.model.model_config
        logger.info(f"model: {type(mc).__name__} hidden={getattr(mc, 'hidden_size', '?')} layers={getattr(mc, 'num_hidden_layers', '?')}")
        if self.tokens is not None:
            logger.info(f"global batch size: {human_format(self.global_batch_size_in_tokens)} tokens")


def model_config_from_dict(d: dict):
    """Pick the model config class from the discriminator key; plain dicts default to Qwen2 (like the reference)."""
    if d.get("is_llama_config"):
        return from_dict(LlamaConfig, d)
    if d.get("is_starcoder2_config"):
        return from_dict(Starcoder2Config, d)
    return from_dict(Qwen2Config, d)


def _declared_model_config_class(config_class: Type) -> Optional[Type]:
    """The dataclass a ``Config`` subclass declares for ``model.model_config`` (None when it keeps the stock union), so that
    an extended config round-trips through YAML without the caller naming the class again."""
    import dataclasses
    import typing

    def concrete(tp):
        if typing.get_origin(tp) is Union:
            args = [a for a in typing.get_args(tp) if a is not type(None)]
            tp = args[0] if len(args) == 1 else None
        return tp if (isinstance(tp, type) and dataclasses.is_dataclass(tp)) else None

    try:
        model_args = concrete(typing.get_type_hints(config_class).get("model"))
        if model_args is None or model_args is ModelArgs:
            return None
        return concrete(typing.get_type_hints(model_args).get("model_config"))
    except Exception:
        return None


_LEGACY_ADAM_KEYS = ("adam_beta1", "adam_beta2", "adam_eps", "torch_adam_is_fused")


def upgrade_legacy_config_dict(config_dict: dict) -> dict:
    """Rewrite spellings that older configuration files of the reference use into the current schema (a copy is returned; a
    warning names every rewrite).  Several of the reference's own example files are still written this way
    (examples/mup/configs/*.yaml, examples/config_nanoset.yaml, examples/config_resume_training.yaml):

    * AdamW settings directly under ``optimizer`` instead of under ``optimizer.optimizer_factory``;
    * ``dataset_folder`` as a mapping ``{folder: weight}`` instead of ``dataset_folder`` + ``dataset_weights`` lists;
    * ``interleaved_rotary`` for ``rope_interleaved`` in a model configuration."""
    import copy
    import warnings

    d = copy.deepcopy(config_dict)
    opt = d.get("optimizer")
    if isinstance(opt, dict) and "optimizer_factory" not in opt and any(k in opt for k in _LEGACY_ADAM_KEYS):
        opt["optimizer_factory"] = {"name": "adamW", **{k: opt.pop(k) for k in _LEGACY_ADAM_KEYS if k in opt}}
        warnings.warn("config: AdamW settings directly under `optimizer` moved to `optimizer.optimizer_factory`")
    for stage in d.get("data_stages") or []:
        dataset = (stage.get("data") or {}).get("dataset") if isinstance(stage, dict) else None
        if isinstance(dataset, dict) and isinstance(dataset.get("dataset_folder"), dict):
            mapping = dataset["dataset_folder"]
            dataset["dataset_folder"], dataset["dataset_weights"] = list(mapping.keys()), [float(w) for w in mapping.values()]
            warnings.warn("config: `dataset_folder` given as {folder: weight} split into `dataset_folder` and `dataset_weights`")
    model_config = (d.get("model") or {}).get("model_config") if isinstance(d.get("model"), dict) else None
    if isinstance(model_config, dict) and "interleaved_rotary" in model_config:
        model_config.setdefault("rope_interleaved", model_config.pop("interleaved_rotary"))
        warnings.warn("config: `interleaved_rotary` renamed to `rope_interleaved`")
    return d


def get_config_from_dict(config_dict: dict, config_class: Type = Config, skip_unused_config_keys: bool = False, skip_null_keys: bool = False, model_config_class: Optional[Type] = None):
    config_dict = upgrade_legacy_config_dict(config_dict)
    if skip_unused_config_keys:
        known = {f.name for f in fields(config_class)}
        config_dict = {k: v for k, v in config_dict.items() if k in known}
    if skip_null_keys:
        config_dict = {k: ({kk: vv for kk, vv in v.items() if vv is not None} if isinstance(v, dict) else v) for k, v in config_dict.items() if v is not None}
    config_dict = dict(config_dict)
    # resolve the model config by discriminator before the strict loader sees the Union
    model = config_dict.get("model")
    if model_config_class is None:
        model_config_class = _declared_model_config_class(config_class)
    if isinstance(model, dict) and isinstance(model.get("model_config"), dict):
        model = dict(model)
        raw = model["model_config"]
        model["model_config"] = from_dict(model_config_class, raw) if model_config_class is not None else model_config_from_dict(raw)
        config_dict["model"] = model
    return from_dict(config_class, config_dict, strict=True)


def get_config_from_file(config_path: str, config_class: Type = Config, model_config_class: Optional[Type] = None, skip_unused_config_keys: bool = False, skip_null_keys: bool = False) -> Config:
    with open(config_path) as f:
        config_dict = yaml.load(f, Loader=SafeLoader)
    return get_config_from_dict(config_dict, config_class=config_class, skip_unused_config_keys=skip_unused_config_keys, skip_null_keys=skip_null_keys, model_config_class=model_config_class)
