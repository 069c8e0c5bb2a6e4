"""Thin layer over ``torch.distributed`` used everywhere in the framework.

Differences from the reference wrapper (reference src/nanotron/distributed.py:1-280):

* both ``nccl`` (GPU) and ``gloo`` (CPU) are first class, so every multi-rank code
  path can be exercised without a GPU;
* the coalesced helpers work on *flat views* whenever the caller hands tensors that
  already live back to back in one buffer (the common case here, since gradients and
  parameters are stored in flat buffers), so no flatten/unflatten copy is done;
* size-1 groups are a no-op instead of an assertion.
"""
from __future__ import annotations

import datetime
import os
from functools import cache, lru_cache
from typing import List, Optional, Sequence

import torch
import torch.distributed as torch_dist
from torch.distributed import *  # noqa: F401,F403  (re-export, like the reference does)
from torch.distributed import ProcessGroup, ReduceOp, Work  # noqa: F401

default_pg_timeout = datetime.timedelta(minutes=20)


def new_group(ranks=None, timeout=default_pg_timeout, backend=None, pg_options=None) -> ProcessGroup:
    if len(ranks) == 0:
        raise ValueError("Cannot create a group with no ranks inside it")
    return torch_dist.new_group(ranks=list(map(int, ranks)), timeout=timeout, backend=backend, pg_options=pg_options)


def _is_flat_contiguous(tensors: Sequence[torch.Tensor]) -> bool:
    """True when ``tensors`` are consecutive slices of a single storage with the same dtype."""
    if len(tensors) == 0:
        return False
    first = tensors[0]
    if not all(t.is_contiguous() and t.dtype == first.dtype and t.device == first.device for t in tensors):
        return False
    base = first.untyped_storage().data_ptr()
    if any(t.untyped_storage().data_ptr() != base for t in tensors):
        return False
    expected = first.data_ptr()
    for t in tensors:
        if t.data_ptr() != expected:
            return False
        expected += t.numel() * t.element_size()
    return True


def _flat_view(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    first = tensors[0]
    total = sum(t.numel() for t in tensors)
    return torch.as_strided(first, (total,), (1,), storage_offset=first.storage_offset())


def reduce_scatter_tensor(output, input, op=ReduceOp.SUM, group=None, async_op=False) -> Optional[Work]:
    if group is not None and group.size() == 1:
        output.copy_(input.view_as(output))
        return None
    return torch_dist.reduce_scatter_tensor(output, input, op=op, group=group, async_op=async_op)


def all_gather_into_tensor(output_tensor, input_tensor, group=None, async_op=False) -> Optional[Work]:
    if group is not None and group.size() == 1:
        output_tensor.copy_(input_tensor.view_as(output_tensor))
        return None
    return torch_dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)


def all_reduce_coalesced(tensors: List[torch.Tensor], op=ReduceOp.SUM, group=None, async_op=False):
    """All-reduce a list of tensors with one collective (flat view when possible, else a packed copy)."""
    if len(tensors) == 0:
        return None
    if group is not None and group.size() == 1:
        return None
    if _is_flat_contiguous(tensors):
        return torch_dist.all_reduce(_flat_view(tensors), op=op, group=group, async_op=async_op)
    by_dtype = {}
    for t in tensors:
        by_dtype.setdefault(t.dtype, []).append(t)
    for ts in by_dtype.values():
        flat = torch.cat([t.reshape(-1) for t in ts])
        torch_dist.all_reduce(flat, op=op, group=group)
        offset = 0
        for t in ts:
            t.copy_(flat[offset : offset + t.numel()].view_as(t))
            offset += t.numel()
    return None


def reduce_scatter_coalesced(
    output_tensor_list: List[torch.Tensor],
    input_tensor_lists: List[List[torch.Tensor]],
    op=ReduceOp.SUM,
    group=None,
    async_op=False,
):
    """``output_tensor_list[i] = reduce_r input_tensor_lists[i][my_rank]`` for every i, with one collective per dtype."""
    assert not async_op, "async reduce_scatter_coalesced is not supported"
    world = get_world_size(group)
    rank = torch_dist.get_rank(group)
    if world == 1:
        for out, ins in zip(output_tensor_list, input_tensor_lists):
            out.copy_(ins[0])
        return None
    assert all(len(ins) == world for ins in input_tensor_lists)
    # pack per destination rank
    per_rank = [torch.cat([ins[r].reshape(-1) for ins in input_tensor_lists]) for r in range(world)]
    sizes = {p.numel() for p in per_rank}
    assert len(sizes) == 1, "every rank must receive the same number of elements"
    out_flat = torch.empty_like(per_rank[rank])
    torch_dist.reduce_scatter(out_flat, per_rank, op=op, group=group)
    offset = 0
    for out in output_tensor_list:
        out.copy_(out_flat[offset : offset + out.numel()].view_as(out))
        offset += out.numel()
    return None


def all_gather_coalesced(
    output_tensor_lists: List[List[torch.Tensor]],
    input_tensor_list: List[torch.Tensor],
    group=None,
    async_op=False,
):
    """``output_tensor_lists[i][r] = input_tensor_list[i] of rank r``; slices may differ in size between ranks."""
    assert not async_op
    world = get_world_size(group)
    if world == 1:
        for outs, inp in zip(output_tensor_lists, input_tensor_list):
            if outs[0].data_ptr() != inp.data_ptr():
                outs[0].copy_(inp)
        return None
    rank = torch_dist.get_rank(group)
    recv = [torch.cat([outs[r].reshape(-1) for outs in output_tensor_lists]) if len(output_tensor_lists) else None for r in range(world)]
    send = torch.cat([t.reshape(-1) for t in input_tensor_list])
    assert recv[rank].numel() == send.numel()
    torch_dist.all_gather(recv, send, group=group)
    for r in range(world):
        offset = 0
        for outs in output_tensor_lists:
            n = outs[r].numel()
            outs[r].copy_(recv[r][offset : offset + n].view_as(outs[r]))
            offset += n
    return None


def get_world_size(group=None) -> int:
    return torch_dist.get_world_size(group)


@cache
def get_global_rank(group: ProcessGroup, group_rank: int) -> int:
    """Cached: this sits on the pipeline hot path (called per send/recv)."""
    if group is None:
        return group_rank
    return torch_dist.get_global_rank(group, group_rank)


def get_global_ranks(group: ProcessGroup):
    return tuple(sorted(get_global_rank(group, i) for i in range(group.size())))


@lru_cache
def get_rank(group: Optional[ProcessGroup] = None) -> int:
    """Cached rank lookup that raises (instead of returning -1) when the caller is outside ``group``."""
    result = torch_dist.get_rank(group)
    if result == -1:
        raise RuntimeError("Can not call `get_rank` on a group in which current process is not a part of")
    return result


def initialize_torch_distributed(backend: Optional[str] = None) -> bool:
    """env:// rendezvous. ``backend`` defaults to nccl when CUDA is present, gloo otherwise."""
    rank = int(os.getenv("RANK", "0"))
    world_size = int(os.getenv("WORLD_SIZE", "1"))
    local_rank = int(os.getenv("LOCAL_RANK", "0"))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        if not torch.cuda.is_available():
            raise RuntimeError("nccl backend requested but CUDA is not available")
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", local_rank % torch.cuda.device_count())
    torch_dist.init_process_group(
        init_method="env://", world_size=world_size, rank=rank, backend=backend, timeout=default_pg_timeout, **kwargs
    )
    get_rank.cache_clear()
    get_global_rank.cache_clear()
    return True
