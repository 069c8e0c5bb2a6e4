"""Where a tensor lives inside a checkpoint, and how shards written under one tensor-parallel size are re-cut for another.

The file-name grammar is the checkpoint format itself and is kept byte for byte (format parity: reference
src/nanotron/serialize/utils.py):

    a.b.weight  ->  a/b/<kind>_weight.safetensors                                              whole tensor
                    a/b/<kind>_weight_pp-rank-P-of-NP_tp-rank-T-of-NT.safetensors              sharded over tp
                    a/b/<kind>_weight_pp-rank-P-of-NP_tp-rank-T-of-NT_exp-rank-E-of-NE.safetensors   sharded over experts too

``shard_file_name`` builds the last component, ``parse_shard_file_name`` reads it back (the resharding loader needs to know
which pipeline / tensor / expert rank wrote a file it finds on disk).
"""
from __future__ import annotations

import re
from enum import Enum
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import SlicesPair

RankAndSize = Tuple[int, int]

_SHARD_RE = re.compile(r"pp-rank-(?P<pp>\d+)-of-(?P<pp_size>\d+)_tp-rank-(?P<tp>\d+)-of-(?P<tp_size>\d+)(?:_exp-rank-(?P<exp>\d+)-of-(?P<exp_size>\d+))?")


class ObjectType(Enum):
    MODEL = "model"
    OPTIMIZER = "optimizer"
    LR_SCHEDULER = "lr_scheduler"


def get_exp_tp_pp_rank_and_size_from(world_rank: int, parallel_context: ParallelContext) -> Tuple[RankAndSize, RankAndSize, RankAndSize]:
    """((expert rank, size), (tp rank, size), (pp rank, size)) of a global rank: the triple ``get_path`` takes."""
    local = parallel_context.get_local_ranks(world_rank=world_rank)
    sizes = {"ep": parallel_context.expert_parallel_size, "tp": parallel_context.tensor_parallel_size, "pp": parallel_context.pipeline_parallel_size}
    return tuple((local[axis], sizes[axis]) for axis in ("ep", "tp", "pp"))


def shard_file_name(kind: ObjectType, leaf: str, ranks: Optional[Tuple[RankAndSize, RankAndSize, RankAndSize]], is_expert_sharded: bool) -> str:
    parts = [f"{kind.value}_{leaf}"]
    if ranks:
        (exp_rank, exp_size), (tp_rank, tp_size), (pp_rank, pp_size) = ranks
        parts.append(f"pp-rank-{pp_rank}-of-{pp_size}")
        parts.append(f"tp-rank-{tp_rank}-of-{tp_size}")
        if is_expert_sharded and exp_size != 1:
            parts.append(f"exp-rank-{exp_rank}-of-{exp_size}")
    return "_".join(parts) + ".safetensors"


def parse_shard_file_name(path) -> Optional[Dict[str, int]]:
    """{"pp", "pp_size", "tp", "tp_size"[, "exp", "exp_size"]} of a shard file, or None for a whole-tensor file."""
    m = _SHARD_RE.search(str(path))
    return None if m is None else {k: int(v) for k, v in m.groupdict().items() if v is not None}


def get_path(tensor_name: str, type: ObjectType, exp_tp_pp_rank_and_size: Optional[Tuple[RankAndSize, RankAndSize, RankAndSize]], is_expert_sharded: bool, prefix: Optional[Path] = None):
    """Path components (or, with ``prefix``, the full path) of the file that holds ``tensor_name``."""
    *folders, leaf = tensor_name.split(".")
    components = folders + [shard_file_name(type, leaf, exp_tp_pp_rank_and_size, is_expert_sharded)]
    return components if prefix is None else Path(prefix).joinpath(*components)


def extract_tp_pp_rank_from_shard_path(shard_path: Path):
    """(pp rank, tp rank) of a shard file, as strings (they key the shard-metadata tables)."""
    found = parse_shard_file_name(shard_path)
    return str(found["pp"]), str(found["tp"])


def merge_and_shard_tp_tensors(buffer: torch.Tensor, unsharded_buffer: torch.Tensor, shards_and_slices_maps: List[Tuple[torch.Tensor, Tuple[SlicesPair, ...]]], shard_metadata) -> torch.Tensor:
    """Scatter every stored shard into ``unsharded_buffer`` (each with the slices it was written with), then gather from it the
    slices this rank's shard is made of under the new layout."""
    for stored, written_as in shards_and_slices_maps:
        for piece in written_as:
            unsharded_buffer[piece.global_slices] = stored[piece.local_slices]
    for piece in shard_metadata.local_global_slices_pairs:
        buffer[piece.local_slices] = unsharded_buffer[piece.global_slices]
    return buffer
