"""Helpers that turn a locally allocated shard into a sharded ``NanotronParameter``.

Parity: reference src/nanotron/parallel/sharded_parameters.py:11-116.  ``contiguous_chunks`` describes fused
projections (q|k|v or gate|up): each chunk is split evenly across the group, so the local tensor is the
concatenation of this rank's slice of every chunk.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import numpy as np
from torch import nn

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.parameters import NanotronParameter, SlicesPair


@dataclasses.dataclass
class SplitConfig:
    split_dim: int
    contiguous_chunks: Optional[Tuple[int, ...]] = None  # sizes along split_dim in the *unsharded* tensor


def create_sharded_parameter(parameter: nn.Parameter, global_ranks: Tuple[int, ...], local_global_slices_pairs: Tuple[SlicesPair, ...], unsharded_shape: Tuple[int, ...]) -> NanotronParameter:
    if not isinstance(parameter, NanotronParameter):
        parameter = NanotronParameter(tensor=parameter, requires_grad=parameter.requires_grad)
    parameter.mark_as_sharded(global_ranks=global_ranks, local_global_slices_pairs=local_global_slices_pairs, unsharded_shape=unsharded_shape)
    return parameter


def compute_slices_pairs(local_shape, split_config: SplitConfig, rank: int, world_size: int):
    """Return (pairs, unsharded_shape) for a tensor of ``local_shape`` held by ``rank`` of ``world_size``."""
    ndim = len(local_shape)
    dim = split_config.split_dim
    unsharded_shape = tuple(s * world_size if i == dim else s for i, s in enumerate(local_shape))
    if split_config.contiguous_chunks is None:
        n = local_shape[dim]
        g = tuple(slice(rank * n, (rank + 1) * n) if i == dim else slice(None) for i in range(ndim))
        l = tuple(slice(None) for _ in range(ndim))
        return (SlicesPair(local_slices=l, global_slices=g),), unsharded_shape
    chunks = split_config.contiguous_chunks
    assert sum(chunks) == unsharded_shape[dim], f"contiguous_chunks {chunks} must sum to the unsharded size {unsharded_shape[dim]}"
    assert all(c % world_size == 0 for c in chunks), f"every chunk of {chunks} must be divisible by the group size {world_size}"
    pairs = []
    g_off, l_off = 0, 0
    for c in chunks:
        per = c // world_size
        g = tuple(slice(g_off + rank * per, g_off + (rank + 1) * per) if i == dim else slice(None) for i in range(ndim))
        l = tuple(slice(l_off, l_off + per) if i == dim else slice(None) for i in range(ndim))
        pairs.append(SlicesPair(local_slices=l, global_slices=g))
        g_off += c
        l_off += per
    return tuple(pairs), unsharded_shape


def create_sharded_parameter_from_config(parameter: nn.Parameter, pg: dist.ProcessGroup, split_config: SplitConfig) -> NanotronParameter:
    rank = dist.get_rank(pg)
    world = pg.size()
    pairs, unsharded_shape = compute_slices_pairs(tuple(parameter.shape), split_config, rank, world)
    return create_sharded_parameter(parameter, global_ranks=dist.get_global_ranks(pg), local_global_slices_pairs=pairs, unsharded_shape=unsharded_shape)


def mark_all_parameters_in_module_as_sharded(module: nn.Module, pg: dist.ProcessGroup, split_config: SplitConfig):
    """Replace every direct or nested plain parameter of ``module`` by a sharded ``NanotronParameter``."""
    for sub in module.modules():
        for name, param in list(sub.named_parameters(recurse=False)):
            setattr(sub, name, create_sharded_parameter_from_config(parameter=param, pg=pg, split_config=split_config))
