"""Gradient averaging when expert parallelism is laid over the data-parallel axis.

With ``ep`` expert-parallel ranks inside a data-parallel group of ``dp`` ranks, an expert's weights exist once per
``expert_dp = dp / ep`` ranks, yet their gradient already contains the tokens of all ``ep`` ranks that were dispatched to it.
Dense weights are ordinary replicas over ``dp x cp``.  Both kinds must end up as the mean over the same ``dp x cp`` micro-batches:

    dense  : sum over dp x cp, divided by dp x cp
    expert : sum over expert_dp (and cp), divided by dp x cp          (the sum over ep happened in the dispatch)

The reference has no expert parallelism in its core (its MoE layer never communicates), so this has no counterpart there.
"""
from __future__ import annotations

from typing import Iterable

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.data_parallel.utils import average_gradients


def is_expert_parameter(param, parallel_context) -> bool:
    """True for parameters sharded over the expert-parallel axis (each ep rank holds different experts)."""
    return bool(getattr(param, "is_sharded", False)) and param.get_sharded_info().is_expert_sharded(parallel_context)


def sync_dense_and_expert_gradients(dense: Iterable[torch.Tensor], experts: Iterable[torch.Tensor], parallel_context) -> None:
    ctx = parallel_context
    replicas = ctx.dp_cp_pg.size()
    dense, experts = list(dense), list(experts)
    if dense and replicas > 1:
        average_gradients(dense, ctx.dp_cp_pg)
    if experts:
        if ctx.expert_dp_pg.size() > 1:
            dist.all_reduce_coalesced(experts, op=dist.ReduceOp.SUM, group=ctx.expert_dp_pg)
        if ctx.cp_pg.size() > 1:
            dist.all_reduce_coalesced(experts, op=dist.ReduceOp.SUM, group=ctx.cp_pg)
        if replicas > 1:
            torch._foreach_div_(experts, replicas)
