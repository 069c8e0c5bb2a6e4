"""Parameters shared by several ranks or several modules, and the synchronisation of their gradients.

Parity: reference src/nanotron/parallel/tied_parameters.py:18-167.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

from torch import nn

import nanotron_b200.distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.utils import get_parameter_and_parent_module

logger = get_logger(__name__)


def create_tied_parameter(parameter: nn.Parameter, name: str, global_ranks: Tuple[int, ...], reduce_op, root_module: nn.Module) -> NanotronParameter:
    if not isinstance(parameter, NanotronParameter):
        parameter = NanotronParameter(tensor=parameter, requires_grad=parameter.requires_grad)
    parameter.mark_as_tied(name=name, global_ranks=global_ranks, reduce_op=reduce_op, root_module=root_module)
    return parameter


def tie_parameters(root_module: nn.Module, ties: List[Tuple[str, Tuple[int, ...]]], parallel_context, reduce_op):
    """Tie the listed ``(target name, global ranks)``.  Ties must stay inside one data-parallel replica; targets living
    on this process end up sharing a single ``NanotronParameter`` object."""
    if len(ties) < 1:
        raise ValueError("Can't tie nothing")
    dp_ranks = tuple(
        sorted({parallel_context.get_local_ranks(world_rank=r)["dp"] for _, ranks in ties for r in ranks})
    )
    assert len(dp_ranks) == 1, f"Tying weights has to happen with a replica of a model. Got the ranks from the following replicas: {dp_ranks}"
    all_ranks = tuple(sorted({r for _, ranks in ties for r in ranks}))
    me = dist.get_rank(parallel_context.world_pg)
    new_param = None
    for target, ranks in ties:
        if me not in ranks:
            continue
        param, parent, attr = get_parameter_and_parent_module(target, root_module)
        if new_param is None:
            new_param = create_tied_parameter(param, name=target, global_ranks=all_ranks, reduce_op=reduce_op, root_module=root_module)
        setattr(parent, attr, new_param)


def create_pg_for_tied_weights(root_module: nn.Module, parallel_context):
    """Make sure a process group exists for every distinct set of ranks that share a tied parameter.
    Collective over the world group: every rank learns every set, then all ranks create the groups in sorted order."""
    local = sorted({tuple(sorted(p.get_tied_info().global_ranks)) for p in root_module.parameters() if isinstance(p, NanotronParameter) and p.is_tied})
    gathered: List[Optional[list]] = [None] * parallel_context.world_pg.size()
    dist.all_gather_object(gathered, local, group=parallel_context.world_pg)
    for ranks in sorted({tuple(g) for per_rank in gathered for g in per_rank}):
        if ranks not in parallel_context.world_ranks_to_pg:
            parallel_context.world_ranks_to_pg[ranks] = dist.new_group(ranks=list(ranks), backend=dist.get_backend())


def get_tied_id_to_param(parameters: List[NanotronParameter], root_module: nn.Module) -> Dict[Tuple[str, Tuple[int, ...]], NanotronParameter]:
    module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in root_module.named_modules()}
    module_id_to_prefix[id(root_module)] = ""
    out = {}
    for p in parameters:
        if not (isinstance(p, NanotronParameter) and p.is_tied):
            continue
        info = p.get_tied_info()
        out[(info.get_full_name_from_module_id_to_prefix(module_id_to_prefix), info.global_ranks)] = p
    return out


def sync_tied_weights_gradients(module: nn.Module, parallel_context, grad_accumulator=None):
    """All-reduce the gradient of every tied parameter over its tie group (one coalesced collective per group/op)."""
    named = sorted(get_tied_id_to_param(list(module.parameters()), root_module=module).items(), key=lambda x: x[0])
    group_to_grads: "OrderedDict[Tuple, List]" = OrderedDict()
    for (name, ranks), param in named:
        info = param.get_tied_info()
        if info.reduce_op is None or len(ranks) <= 1:
            continue
        grad = grad_accumulator.get_grad_buffer(name=name) if grad_accumulator is not None else param.grad
        assert grad is not None, f"Tied parameter {name} has no gradient"
        key = (tuple(sorted(ranks)), info.reduce_op)
        group_to_grads.setdefault(key, []).append(grad)
    for (ranks, op), grads in group_to_grads.items():
        dist.all_reduce_coalesced(grads, op=op, group=parallel_context.world_ranks_to_pg[ranks])
