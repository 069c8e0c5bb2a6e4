"""Parameter (de)serialisation: one safetensors file per parameter shard, tensor key ``"data"``, shard geometry in the
file's string metadata (format parity: reference src/nanotron/serialize/weights.py:30-394).

Loading is topology agnostic: if the file for this rank's coordinates exists it is read directly; otherwise all
shards of the parameter are merged through their slice maps and re-cut for the current tensor-parallel size.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
from packaging.version import Version
from safetensors.torch import safe_open, save_file
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.constants import CHECKPOINT_VERSION
from nanotron_b200.logging import log_rank
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter, ShardedInfo, SlicesPair
from nanotron_b200.serialize.metadata import CheckpointMetadata, TensorMetadata, load_meta
from nanotron_b200.serialize.utils import ObjectType, extract_tp_pp_rank_from_shard_path, get_exp_tp_pp_rank_and_size_from, get_path, merge_and_shard_tp_tensors

logger = logging.get_logger(__name__)


def save_weights(model: nn.Module, parallel_context: ParallelContext, root_folder: Path):
    root_folder = Path(root_folder) / "model"
    # only one data-parallel (x context-parallel) replica writes; experts are written by every expert-parallel rank
    dp_cp_rank = dist.get_rank(parallel_context.dp_cp_pg)
    ep_size = parallel_context.expert_parallel_size
    ep_rank = dist.get_rank(parallel_context.ep_pg) if ep_size > 1 else 0
    expert_dp_rank = dist.get_rank(parallel_context.expert_dp_pg) if ep_size > 1 else dp_cp_rank
    module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in model.named_modules()}
    module_id_to_prefix[id(model)] = ""
    for name, param_or_buffer in model.state_dict().items():
        try:
            param = model.get_parameter(name)
        except AttributeError:
            param = None
        is_expert = False
        if isinstance(param, NanotronParameter) and param.is_sharded:
            is_expert = param.get_sharded_info().is_expert_sharded(parallel_context)
        if is_expert:
            cp_rank = dist.get_rank(parallel_context.cp_pg)
            if expert_dp_rank != 0 or cp_rank != 0:
                continue
        elif dp_cp_rank != 0:
            continue
        if isinstance(param, NanotronParameter):
            metadata: Dict[str, str] = {}
            if param.is_tied:
                tied_info = param.get_tied_info()
                base_name = tied_info.get_full_name_from_module_id_to_prefix(module_id_to_prefix=module_id_to_prefix)
                group_ranks = tied_info.global_ranks
                group = parallel_context.world_ranks_to_pg[tuple(sorted(group_ranks))]
                # only the first rank of the tie group writes
                if dist.get_rank(group) != 0:
                    continue
            else:
                base_name = name
            if param.is_sharded:
                sharded_info: ShardedInfo = param.get_sharded_info()
                group = parallel_context.world_ranks_to_pg[tuple(sorted(sharded_info.global_ranks))]
                exp_tp_pp = get_exp_tp_pp_rank_and_size_from(world_rank=dist.get_global_rank(group, dist.get_rank(group)), parallel_context=parallel_context)
                metadata = TensorMetadata(version=CHECKPOINT_VERSION, local_global_slices_pairs=sharded_info.local_global_slices_pairs, unsharded_shape=sharded_info.unsharded_shape).to_str_dict()
            else:
                exp_tp_pp = None
            path = get_path(base_name, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=exp_tp_pp, is_expert_sharded=is_expert, prefix=root_folder)
            path.parent.mkdir(exist_ok=True, parents=True)
            try:
                save_file(tensors={"data": param_or_buffer.detach().contiguous().cpu() if param_or_buffer.device.type != "cpu" else param_or_buffer.detach().contiguous()}, filename=path, metadata=metadata)
            except Exception as e:
                log_rank(f"Error saving {path} with {metadata}", logger=logger, level=logging.ERROR, rank=0)
                raise e
        else:
            raise NotImplementedError(f"Parameters {name} should be a NanotronParameter")


class CheckpointVersionFromShardFileException(Exception):
    """Raised when a shard file carries no version (files written before v1.2)."""


def read_checkpoint_version_from_shard_file(param_save_path: Path) -> Version:
    try:
        with safe_open(param_save_path, framework="pt", device="cpu") as fi:
            return TensorMetadata.from_str_dict(fi.metadata()).version
    except (KeyError, TypeError, AssertionError):
        raise CheckpointVersionFromShardFileException()


def read_checkpoint_version_from_meta(parallel_context: ParallelContext, root_folder: Path) -> Version:
    return load_meta(parallel_context=parallel_context, root_folder=root_folder).version


def get_checkpoint_version(parallel_context, root_folder, param_save_path: Path) -> Version:
    try:
        return read_checkpoint_version_from_shard_file(param_save_path)
    except CheckpointVersionFromShardFileException:
        return read_checkpoint_version_from_meta(parallel_context, root_folder)


def load_sharded_param_latest(param_or_buffer: torch.Tensor, sharded_info: ShardedInfo, shards_path: List[Path], param_shard_metadata: Optional[dict] = None):
    """Fill ``param_or_buffer`` (this rank's shard) from all stored shards of the parameter."""
    shards_and_slices_maps: List[Tuple[torch.Tensor, Tuple[SlicesPair, ...]]] = []
    checkpoint_unsharded_shape = None
    for shard_path in shards_path:
        with safe_open(shard_path, framework="pt", device=str(param_or_buffer.device)) as fi:
            meta = TensorMetadata.from_str_dict(fi.metadata())
            shards_and_slices_maps.append((fi.get_tensor("data"), meta.local_global_slices_pairs))
            if checkpoint_unsharded_shape is None:
                checkpoint_unsharded_shape = meta.unsharded_shape
            else:
                assert checkpoint_unsharded_shape == meta.unsharded_shape, f"Shards of {shard_path} disagree on the unsharded shape"
            if param_shard_metadata is not None:
                pp_rank, tp_rank = extract_tp_pp_rank_from_shard_path(shard_path)
                param_shard_metadata[(pp_rank, tp_rank)] = meta
    assert checkpoint_unsharded_shape is not None, f"no shard found among {shards_path}"
    assert tuple(checkpoint_unsharded_shape) == tuple(sharded_info.unsharded_shape), f"Shape mismatch: checkpoint {tuple(checkpoint_unsharded_shape)} vs model {tuple(sharded_info.unsharded_shape)}"
    unsharded = torch.empty(tuple(checkpoint_unsharded_shape), dtype=param_or_buffer.dtype, device=param_or_buffer.device)
    merge_and_shard_tp_tensors(buffer=param_or_buffer, unsharded_buffer=unsharded, shards_and_slices_maps=shards_and_slices_maps, shard_metadata=sharded_info)
    return unsharded


def _forget_quantised_copies():
    """Weights were overwritten in place: cached fp8 copies of them (fp8 linear mode) are stale."""
    import sys

    mod = sys.modules.get("nanotron_b200.fp8.parameter")
    if mod is not None:
        mod.weight_cache.invalidate()


def load_weights(model: nn.Module, parallel_context: ParallelContext, root_folder: Path, filtered_state_dict: Optional[Dict[str, Any]] = None):
    """Load parameters in place.  ``filtered_state_dict`` restricts which entries are loaded (name -> tensor)."""
    param_root_folder = Path(root_folder) / "model"
    module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in model.named_modules()}
    module_id_to_prefix[id(model)] = ""
    checkpoint_version: Optional[Version] = None
    state = filtered_state_dict if filtered_state_dict is not None else model.state_dict()
    param_shard_metadata = {}
    for name, param_or_buffer in state.items():
        param_shard_metadata[name] = {}
        try:
            param = model.get_parameter(name)
        except AttributeError:
            param = None
        if not isinstance(param, NanotronParameter):
            raise NotImplementedError(f"Parameters {name} should be a NanotronParameter")
        base_name = param.get_tied_info().get_full_name_from_module_id_to_prefix(module_id_to_prefix) if param.is_tied else name
        if param.is_sharded:
            sharded_info = param.get_sharded_info()
            is_expert = sharded_info.is_expert_sharded(parallel_context)
            group = parallel_context.world_ranks_to_pg[tuple(sorted(sharded_info.global_ranks))]
            exp_tp_pp = get_exp_tp_pp_rank_and_size_from(world_rank=dist.get_global_rank(group, dist.get_rank(group)), parallel_context=parallel_context)
        else:
            sharded_info, is_expert, exp_tp_pp = None, False, None
        path = get_path(base_name, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=exp_tp_pp, prefix=param_root_folder, is_expert_sharded=is_expert)
        if not path.exists() and param.is_tied and hasattr(model, "get_embeddings_lm_head_tied_names"):
            # a tie across pipeline stages joins parameters with different names (embedding / lm head) and only the first rank
            # of the tie group writes, under ITS name: the other members read that file
            for other in model.get_embeddings_lm_head_tied_names():
                alt = get_path(other, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=exp_tp_pp, prefix=param_root_folder, is_expert_sharded=is_expert)
                if other != base_name and (alt.exists() or alt.parent.exists()):
                    base_name, path = other, alt
                    break
        if path.exists():
            with safe_open(path, framework="pt", device=str(param_or_buffer.device)) as fi:
                if param.is_sharded:
                    meta = TensorMetadata.from_str_dict(fi.metadata())
                    param_shard_metadata[name][(str(exp_tp_pp[2][0]), str(exp_tp_pp[1][0]))] = meta
                with torch.no_grad():
                    param_or_buffer.copy_(fi.get_tensor("data"))
        elif not path.parent.exists():
            raise ValueError(f"Checkpoint is empty or checkpoint structure is not matching the model architecture. Couldn't find folder {path.parent} in checkpoint at {root_folder}")
        else:
            if not param.is_sharded:
                raise ValueError(f"`{name}` is not a sharded parameter and {path} is missing")
            suffix = base_name.rsplit(".", 1)[-1]
            shards_path = sorted(path.parent.glob(f"{ObjectType.MODEL.value}_{suffix}_pp-rank-*-of-*_tp-rank-*-of-*.safetensors"))
            if len(shards_path) == 0:
                raise ValueError(f"Could not find any shards {ObjectType.MODEL.value}_{suffix}*.safetensors in {path.parent}. If you notice `.safetensors` in the middle of the name of some of the checkpoints files. You need to run `scripts/fix_checkpoint_bad_naming.py`.")
            if checkpoint_version is None:
                checkpoint_version = get_checkpoint_version(parallel_context, root_folder, param_save_path=shards_path[0])
            with torch.no_grad():
                load_sharded_param_latest(param_or_buffer=param_or_buffer, sharded_info=sharded_info, shards_path=shards_path, param_shard_metadata=param_shard_metadata[name])
    _forget_quantised_copies()
    return param_shard_metadata


def get_checkpoint_paths_list(model: nn.Module, parallel_context: ParallelContext, root_folder: Path, only_list_folders: bool = False, only_list_current_process: bool = True, filtered_state_dict: Optional[Dict[str, Any]] = None):
    """Paths (or parent folders) of the files ``load_weights`` would read for this process."""
    param_root_folder = Path(root_folder) / "model"
    module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in model.named_modules()}
    module_id_to_prefix[id(model)] = ""
    paths = []
    state = filtered_state_dict if filtered_state_dict is not None else model.state_dict()
    for name in state.keys():
        param = model.get_parameter(name)
        if not isinstance(param, NanotronParameter):
            raise NotImplementedError(f"Parameters {name} should be a NanotronParameter")
        base_name = param.get_tied_info().get_full_name_from_module_id_to_prefix(module_id_to_prefix) if param.is_tied else name
        if param.is_sharded:
            sharded_info = param.get_sharded_info()
            is_expert = sharded_info.is_expert_sharded(parallel_context)
            if only_list_current_process:
                group = parallel_context.world_ranks_to_pg[tuple(sorted(sharded_info.global_ranks))]
                exp_tp_pp = get_exp_tp_pp_rank_and_size_from(world_rank=dist.get_global_rank(group, dist.get_rank(group)), parallel_context=parallel_context)
                path = get_path(base_name, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=exp_tp_pp, prefix=param_root_folder, is_expert_sharded=is_expert)
                paths.append(path.parent if only_list_folders else path)
            else:
                for world_rank in sharded_info.global_ranks:
                    exp_tp_pp = get_exp_tp_pp_rank_and_size_from(world_rank=world_rank, parallel_context=parallel_context)
                    path = get_path(base_name, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=exp_tp_pp, prefix=param_root_folder, is_expert_sharded=is_expert)
                    paths.append(path.parent if only_list_folders else path)
        else:
            path = get_path(base_name, type=ObjectType.MODEL, exp_tp_pp_rank_and_size=None, prefix=param_root_folder, is_expert_sharded=False)
            paths.append(path.parent if only_list_folders else path)
    return list(dict.fromkeys(paths))
