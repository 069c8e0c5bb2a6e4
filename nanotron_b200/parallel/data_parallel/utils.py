"""Gradient averaging over data-parallel replicas for models that do not go through the fused NVLink step
(capability parity: reference src/nanotron/parallel/data_parallel/utils.py:10-52).

There is no ``DistributedDataParallel`` wrapper in this framework, so there is no reducer to trigger: gradients are
averaged once per step, after the last micro-batch, either inside the fp32 gradient accumulator's flat buffer
(``grad_accumulator.sync_gradients_across_dp``) or, without an accumulator, over the parameters' ``.grad`` tensors with
one coalesced all-reduce per dtype.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

import nanotron_b200.distributed as dist


def average_gradients(grads: Iterable[torch.Tensor], group: dist.ProcessGroup, divide_by: Optional[int] = None) -> None:
    """In-place mean of every tensor over ``group`` (sum, then divide by ``divide_by`` or the group size), one coalesced
    all-reduce per dtype."""
    by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    denom = divide_by if divide_by is not None else group.size()
    for same in by_dtype.values():
        if group.size() > 1:
            dist.all_reduce_coalesced(same, op=dist.ReduceOp.SUM, group=group)
        if denom != 1:
            torch._foreach_div_(same, denom)


def sync_gradients_across_dp(module: torch.nn.Module, dp_pg: dist.ProcessGroup, reduce_op: dist.ReduceOp = dist.ReduceOp.AVG, reduce_scatter: bool = False, grad_accumulator=None, **_) -> None:
    """Average the gradients of ``module`` over ``dp_pg``.  With a gradient accumulator the exchange happens on its flat fp32
    buffer (optionally as a reduce-scatter, which is what ZeRO-1 needs); otherwise on the parameters' own gradients."""
    if dp_pg.size() == 1:
        return
    if grad_accumulator is not None:
        grad_accumulator.sync_gradients_across_dp(dp_pg=dp_pg, reduce_op=reduce_op, reduce_scatter=reduce_scatter)
        return
    assert not reduce_scatter, "a reduce-scatter of gradients needs the flat buffer of a gradient accumulator"
    grads = [p.grad for p in module.parameters() if p.grad is not None]
    if reduce_op == dist.ReduceOp.AVG:
        average_gradients(grads, dp_pg)
    else:
        for g in grads:
            dist.all_reduce(g, op=reduce_op, group=dp_pg)
