"""Scratch-buffer pool and first-step parameter sync (parity: reference src/nanotron/parallel/utils.py:13-41)."""
from __future__ import annotations

import functools
import operator
from typing import Dict, Tuple

import torch
from torch import nn

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.tied_parameters import get_tied_id_to_param
from nanotron_b200.utils import Singleton


class MemoryBuffer(metaclass=Singleton):
    """Named, growable scratch buffers reused across calls (e.g. the gathered activations of a column linear)."""

    def __init__(self):
        self.buffer: Dict[Tuple[str, torch.dtype, str], torch.Tensor] = {}

    def get(self, name: str, shape, dtype: torch.dtype = torch.bfloat16, device="cuda") -> torch.Tensor:
        required = functools.reduce(operator.mul, shape, 1)
        key = (name, dtype, str(device))
        buf = self.buffer.get(key)
        if buf is None or buf.numel() < required:
            buf = torch.empty(required, dtype=dtype, device=device, requires_grad=False)
            self.buffer[key] = buf
        return buf[:required].view(shape)

    def clear(self):
        self.buffer.clear()


def initial_sync(model: nn.Module, parallel_context):
    """Average parameters over dp (so replicas start equal) and over every tie group."""
    params = [p for p in model.parameters()]
    by_dtype = {}
    for p in params:
        by_dtype.setdefault(p.dtype, []).append(p.data)
    for ts in by_dtype.values():
        dist.all_reduce_coalesced(ts, op=dist.ReduceOp.AVG if dist.get_backend() == "nccl" else dist.ReduceOp.SUM, group=parallel_context.dp_pg)
        if dist.get_backend() != "nccl":
            for t in ts:
                t.div_(parallel_context.dp_pg.size())
    for (_, ranks), param in sorted(get_tied_id_to_param(params, root_module=model).items(), key=lambda x: x[0]):
        group = parallel_context.world_ranks_to_pg[tuple(sorted(ranks))]
        if group.size() == 1:
            continue
        dist.all_reduce(param.data, op=dist.ReduceOp.SUM, group=group)
        param.data.div_(group.size())
