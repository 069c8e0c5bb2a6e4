"""Whole-checkpoint save / load and checkpoint-path resolution (parity: reference src/nanotron/serialize/main.py)."""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional, cast

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging, optim
from nanotron_b200.config import Config
from nanotron_b200.constants import LATEST_FILE_NAME, MODEL_CONFIG_FILE_NAME
from nanotron_b200.logging import log_rank
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.sanity_checks import assert_tensor_synced_across_pg, check_optim_state_in_sync
from nanotron_b200.serialize.metadata import TrainingMetadata, save_meta
from nanotron_b200.serialize.optimizer import save_lr_scheduler, save_optimizer
from nanotron_b200.serialize.weights import save_weights

logger = logging.get_logger(__name__)


def save(
    config: Config,
    model: nn.Module,
    optimizer: Optional[optim.BaseOptimizer],
    lr_scheduler,
    parallel_context: ParallelContext,
    training_metadata: TrainingMetadata,
    root_folder: Path,
    should_save_config: bool = True,
    should_save_model: bool = True,
    should_save_optimizer: bool = True,
    should_save_lr_scheduler: bool = True,
    sanity_checks: bool = True,
) -> None:
    root_folder = Path(root_folder)
    assert isinstance(training_metadata, TrainingMetadata)
    try:
        if should_save_config:
            if dist.get_rank(parallel_context.world_pg) == 0:
                config.save_as_yaml(root_folder / "config.yaml")
    except Exception as e:
        log_rank(f"Error while saving config: {e}", logger=logger, level=logging.ERROR, rank=0)
        raise e
    try:
        if should_save_model:
            save_weights(model=model, parallel_context=parallel_context, root_folder=root_folder)
    except Exception as e:
        log_rank(f"Error while saving weights checkpoint: {e}", logger=logger, level=logging.ERROR, rank=0)
        raise e
    try:
        if should_save_optimizer and optimizer is not None:
            save_optimizer(optimizer=optimizer, parallel_context=parallel_context, root_folder=root_folder)
    except Exception as e:
        log_rank(f"Error while saving optimizer checkpoint: {e}", logger=logger, level=logging.ERROR, rank=0)
        raise e
    try:
        if should_save_lr_scheduler and lr_scheduler is not None and optimizer is not None:
            save_lr_scheduler(lr_scheduler=lr_scheduler, is_zero=optimizer.inherit_from(optim.ZeroDistributedOptimizer), parallel_context=parallel_context, root_folder=root_folder)
    except Exception as e:
        log_rank(f"Error while saving lr_scheduler checkpoint: {e}", logger=logger, level=logging.ERROR, rank=0)
        raise e
    save_meta(root_folder=root_folder, parallel_context=parallel_context, training_metadata=training_metadata)
    if sanity_checks:
        # replicas must agree on what was just written
        for name, param in sorted(model.named_parameters(), key=lambda x: x[0]):
            assert_tensor_synced_across_pg(tensor=param, pg=parallel_context.dp_cp_pg if not _is_expert(param, parallel_context) else parallel_context.expert_dp_pg, msg=lambda err, name=name: f"{name} are not synced across DP {err}")
        if optimizer is not None and not optimizer.inherit_from(optim.ZeroDistributedOptimizer):
            check_optim_state_in_sync(optimizer.state_dict(), parallel_context.dp_pg)
    dist.barrier(parallel_context.world_pg)


def _is_expert(param, parallel_context) -> bool:
    return isinstance(param, NanotronParameter) and param.is_sharded and param.get_sharded_info().is_expert_sharded(parallel_context)


def load(model: nn.Module, optimizer: optim.BaseOptimizer, lr_scheduler, parallel_context: ParallelContext, root_folder: Path):
    """Load weights, optimizer and scheduler; returns the checkpoint metadata."""
    from nanotron_b200.serialize.metadata import load_meta
    from nanotron_b200.serialize.optimizer import load_lr_scheduler, load_optimizer
    from nanotron_b200.serialize.weights import load_weights

    meta = load_meta(parallel_context=parallel_context, root_folder=root_folder)
    shard_meta = load_weights(model=model, parallel_context=parallel_context, root_folder=root_folder)
    load_optimizer(optimizer=optimizer, parallel_context=parallel_context, root_folder=root_folder, param_shard_metadata=shard_meta, model=model)
    load_lr_scheduler(lr_scheduler=lr_scheduler, is_zero=optimizer.inherit_from(optim.ZeroDistributedOptimizer), parallel_context=parallel_context, root_folder=root_folder)
    return meta


def _read_remote_step(url: str, s5cmd_path=None) -> Optional[int]:
    """The step written in a remote ``latest.txt``, or None when there is no such object.  Read through fsspec when a driver for
    the protocol is installed, else with the same ``s5cmd`` tool that moves the checkpoints (``s5cmd cat``)."""
    from nanotron_b200.s3_checkpoints import fs_open

    try:
        with fs_open(url, mode="r") as fi:
            return int(fi.read())
    except FileNotFoundError:
        return None
    except (ImportError, ValueError, OSError) as e:
        log_rank(f"{url}: not readable through fsspec ({type(e).__name__}); asking s5cmd", logger=logger, level=logging.INFO, rank=0)
    import subprocess

    try:
        done = subprocess.run([str(s5cmd_path) if s5cmd_path is not None else "s5cmd", "cat", url], capture_output=True, text=True, timeout=300)
    except FileNotFoundError as e:
        raise RuntimeError(f"cannot read {url}: neither an fsspec driver for the protocol nor the s5cmd tool is available") from e
    return int(done.stdout.strip()) if done.returncode == 0 and done.stdout.strip().isdigit() else None


def parse_ckpt_path(config: Config, parallel_context: Optional[ParallelContext] = None) -> Optional[Path]:
    """Resolve ``checkpoints.resume_checkpoint_path`` to a concrete step folder.

    Accepts a step folder (contains ``config.yaml`` / ``model_config.json``) or a folder of step folders with a
    ``latest.txt``.  ``s3://`` paths are downloaded first (by the first rank of every node) through ``S3Mover``."""
    load_from_candidate = config.checkpoints.resume_checkpoint_path if config.checkpoints is not None else None
    if load_from_candidate is None:
        return None
    candidate = str(load_from_candidate)
    if candidate.startswith("s3:/"):
        from nanotron_b200.s3_checkpoints import S3Mover, check_path_is_local, fs_open

        s3_path = candidate if candidate.startswith("s3://") else candidate.replace("s3:/", "s3://", 1)
        local = Path(config.checkpoints.checkpoints_path)
        latest_meta = s3_path.rstrip("/") + "/" + LATEST_FILE_NAME
        step = _read_remote_step(latest_meta, config.s3_upload.s5cmd_path if config.s3_upload else None)
        if step is not None:
            s3_path = s3_path.rstrip("/") + f"/{step}"
            local_dir = local / str(step)
        else:  # the path names a step folder itself
            local_dir = local / s3_path.rstrip("/").split("/")[-1]
        mover = S3Mover(local_path=str(local_dir), s3_path=s3_path, s5cmd_numworkers=config.s3_upload.s5cmd_numworkers if config.s3_upload else None, s5cmd_concurrency=config.s3_upload.s5cmd_concurrency if config.s3_upload else None, s5cmd_path=config.s3_upload.s5cmd_path if config.s3_upload else None, dummy=bool(int(os.environ.get("LOCAL_RANK", "0")) != 0))
        mover.distributed_wait_for_completion(parallel_context.world_pg if parallel_context is not None else None)
        mover.start_downloading()
        mover.distributed_wait_for_completion(parallel_context.world_pg if parallel_context is not None else None)
        return local_dir
    path = Path(candidate)
    latest = path / LATEST_FILE_NAME
    if latest.exists():
        with open(latest) as fi:
            step = int(fi.read().strip())
        path = path / str(step)
    elif (path / MODEL_CONFIG_FILE_NAME).exists() or (path / "config.yaml").exists():
        pass
    else:
        log_rank(f"No previous checkpoint found in: {path}\n Initializing from scratch.", logger=logger, level=logging.WARNING, rank=0)
        return None
    log_rank(f"Loading checkpoint from {path}", logger=logger, level=logging.INFO, rank=0)
    return path
