"""Placement of a list of named tensors in one flat buffer, and its even split over data-parallel ranks.

Every parameter starts on a 128-element boundary; the total is padded so that ``world`` equal shards tile it.
Rank r owns the half-open element range ``[r*shard, (r+1)*shard)``; a parameter may straddle shards.  The same
layout is used for the fp32 gradient buffer, the half-precision parameter buffer and (restricted to the owned
range) the fp32 master / optimizer-state buffers, so gradient reduce-scatter, optimizer step and parameter
all-gather are each one operation over a contiguous range.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Tuple

import torch

ALIGN = 128


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class FlatLayout:
    offsets: "OrderedDict[str, int]"
    numels: Dict[str, int]
    total: int  # padded
    world: int

    @classmethod
    def build(cls, named_shapes: Iterable[Tuple[str, int]], world: int = 1) -> "FlatLayout":
        offsets, numels, total = OrderedDict(), {}, 0
        for name, n in named_shapes:
            offsets[name] = total
            numels[name] = n
            total += _round_up(n, ALIGN)
        total = _round_up(max(total, ALIGN), ALIGN * world)
        return cls(offsets=offsets, numels=numels, total=total, world=world)

    @property
    def shard(self) -> int:
        return self.total // self.world

    def shard_range(self, rank: int) -> Tuple[int, int]:
        return rank * self.shard, (rank + 1) * self.shard

    def param_range_on_rank(self, name: str, rank: int) -> Tuple[int, int]:
        """Element range of ``name`` (in the parameter's own flattened index space) that falls in ``rank``'s shard."""
        o, n = self.offsets[name], self.numels[name]
        s, e = self.shard_range(rank)
        lo, hi = max(o, s), min(o + n, e)
        if hi <= lo:
            return (0, 0)
        return (lo - o, hi - o)

    def param_name_to_dp_rank_offsets(self) -> Dict[str, Dict[int, Tuple[int, int]]]:
        out = {}
        for name in self.offsets:
            per = {}
            for r in range(self.world):
                rng = self.param_range_on_rank(name, r)
                if rng[1] > rng[0]:
                    per[r] = rng
            out[name] = per
        return out

    def view(self, buffer: torch.Tensor, name: str, shape=None) -> torch.Tensor:
        o, n = self.offsets[name], self.numels[name]
        v = buffer[o : o + n]
        return v.view(shape) if shape is not None else v


_BUFFER_ALLOCATOR = None


def set_buffer_allocator(fn):
    """``fn(numel, dtype, device) -> zero-filled 1-D tensor`` used for every flat buffer (None: ``torch.zeros``).
    The trainer installs a symmetric-memory allocator here so peers can address the buffers directly."""
    global _BUFFER_ALLOCATOR
    _BUFFER_ALLOCATOR = fn


def alloc_flat(numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    if _BUFFER_ALLOCATOR is not None:
        return _BUFFER_ALLOCATOR(numel, dtype, device)
    return torch.zeros(numel, dtype=dtype, device=device)


def flatten_parameters(named_params: List[Tuple[str, torch.nn.Parameter]], layout: FlatLayout) -> Dict[torch.dtype, torch.Tensor]:
    """Move every parameter into one flat buffer per dtype following ``layout`` (``param.data`` becomes a view).
    Returns the buffers by dtype."""
    by_dtype: Dict[torch.dtype, List[Tuple[str, torch.nn.Parameter]]] = {}
    for name, p in named_params:
        by_dtype.setdefault(p.dtype, []).append((name, p))
    buffers = {}
    for dtype, items in by_dtype.items():
        device = items[0][1].device
        existing = getattr(items[0][1], "_ntb_flat_buffer", None)
        if existing is not None and existing.numel() == layout.total and all(
            getattr(p, "_ntb_flat_buffer", None) is existing and p.data_ptr() == existing.data_ptr() + layout.offsets[name] * existing.element_size() for name, p in items
        ):
            buffers[dtype] = existing  # already flattened with this layout
            continue
        buf = alloc_flat(layout.total, dtype, device)
        with torch.no_grad():
            for name, p in items:
                v = layout.view(buf, name, p.shape)
                v.copy_(p.data)
                p.data = v
                p._ntb_flat_buffer = buf
        buffers[dtype] = buf
    return buffers
