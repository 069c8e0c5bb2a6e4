"""Checkpoint path naming and shard merging (format parity: reference src/nanotron/serialize/utils.py)."""
from __future__ import annotations

import re
from enum import Enum
from pathlib import Path
from typing import List, Optional, Tuple

import torch

from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import SlicesPair


class ObjectType(Enum):
    MODEL = "model"
    OPTIMIZER = "optimizer"
    LR_SCHEDULER = "lr_scheduler"


def get_exp_tp_pp_rank_and_size_from(world_rank: int, parallel_context: ParallelContext) -> Tuple[Tuple[int, int], Tuple[int, int], Tuple[int, int]]:
    r = parallel_context.get_local_ranks(world_rank=world_rank)
    return (
        (r["ep"], parallel_context.expert_parallel_size),
        (r["tp"], parallel_context.tensor_parallel_size),
        (r["pp"], parallel_context.pipeline_parallel_size),
    )


def get_path(tensor_name: str, type: ObjectType, exp_tp_pp_rank_and_size: Optional[Tuple[Tuple[int, int], Tuple[int, int], Tuple[int, int]]], is_expert_sharded: bool, prefix: Optional[Path] = None):
    """``a.b.weight`` -> ``[prefix/]a/b/model_weight[_pp-rank-P-of-N_tp-rank-T-of-M[_exp-rank-E-of-K]].safetensors``."""
    suffix = tensor_name.split(".")
    suffix_path, suffix_name = suffix[:-1], suffix[-1]
    if exp_tp_pp_rank_and_size:
        (exp_rank, exp_size), (tp_rank, tp_size), (pp_rank, pp_size) = exp_tp_pp_rank_and_size
        if not is_expert_sharded or exp_size == 1:
            suffix_name = f"{type.value}_{suffix_name}_pp-rank-{pp_rank}-of-{pp_size}_tp-rank-{tp_rank}-of-{tp_size}.safetensors"
        else:
            suffix_name = f"{type.value}_{suffix_name}_pp-rank-{pp_rank}-of-{pp_size}_tp-rank-{tp_rank}-of-{tp_size}_exp-rank-{exp_rank}-of-{exp_size}.safetensors"
    else:
        suffix_name = f"{type.value}_{suffix_name}.safetensors"
    suffix_path.append(suffix_name)
    if prefix is None:
        return suffix_path
    return Path(prefix).joinpath(*suffix_path)


def extract_tp_pp_rank_from_shard_path(shard_path: Path):
    m = re.search(r"pp-rank-(\d+)-of-\d+_tp-rank-(\d+)-of-\d+", str(shard_path))
    pp_rank, tp_rank = m.groups()
    return pp_rank, tp_rank


def merge_and_shard_tp_tensors(buffer: torch.Tensor, unsharded_buffer: torch.Tensor, shards_and_slices_maps: List[Tuple[torch.Tensor, Tuple[SlicesPair, ...]]], shard_metadata) -> torch.Tensor:
    """Rebuild the unsharded tensor from every stored shard, then cut out what the new topology's shard needs."""
    for shard, slices_pairs in shards_and_slices_maps:
        for sp in slices_pairs:
            unsharded_buffer[sp.global_slices] = shard[sp.local_slices]
    for sp in shard_metadata.local_global_slices_pairs:
        buffer[sp.local_slices] = unsharded_buffer[sp.global_slices]
    return buffer
