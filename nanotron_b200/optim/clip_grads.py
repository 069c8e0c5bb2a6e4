"""Global gradient-norm clipping across model-parallel ranks (parity: reference src/nanotron/optim/clip_grads.py:15-97).

No host synchronisation: the clip coefficient stays on the device.  Tied parameters are counted once (on the first
rank of their tie group).  Under ZeRO-1 with reduce-scattered gradients, pass only this rank's gradient slices and
``extra_reduce_group=dp_pg`` so the squared norms are also summed over the shards.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.optim.gradient_accumulator import FP32GradientAccumulator
from nanotron_b200.parallel.parameters import NanotronParameter


def _local_grads(named_parameters, grad_accumulator):
    world_rank = dist.get_rank() if dist.is_initialized() else 0
    grads = []
    for name, param in named_parameters:
        if isinstance(param, NanotronParameter) and param.is_tied:
            ranks = param.get_tied_info().global_ranks
            if world_rank != sorted(ranks)[0]:
                continue  # counted by the first rank of the tie group
        if grad_accumulator is not None:
            g = grad_accumulator.get_grad_buffer(name)
        else:
            g = param.grad
        if g is not None:
            grads.append(g)
    return grads


@torch.no_grad()
def clip_grad_norm(
    mp_pg: dist.ProcessGroup,
    named_parameters: Iterable[Tuple[str, NanotronParameter]],
    max_norm: float,
    grad_accumulator: Optional[FP32GradientAccumulator],
    norm_type: float = 2.0,
    extra_reduce_group: Optional[dist.ProcessGroup] = None,
    grad_slices: Optional[Iterable[torch.Tensor]] = None,
    scale_slices: Optional[Iterable[torch.Tensor]] = None,
) -> torch.Tensor:
    """Scale gradients so their global norm is at most ``max_norm``.  Returns the norm before clipping (0-dim tensor).

    ``grad_slices``: the tensors whose norm is taken (ZeRO-1: this rank's slices, each tied weight on one rank of its tie group
    only).  ``scale_slices``: the tensors that are scaled; it defaults to ``grad_slices`` but must also hold the copies that the
    norm skipped, or a tied weight would be clipped on one rank of its group and not on the others."""
    named_parameters = list(named_parameters)
    grads = list(grad_slices) if grad_slices is not None else _local_grads(named_parameters, grad_accumulator)
    device = grads[0].device if grads else (named_parameters[0][1].device if named_parameters else torch.device("cpu"))
    if norm_type == math.inf:
        total = torch.stack([g.detach().abs().max().float() for g in grads]).max() if grads else torch.zeros([], device=device)
        dist.all_reduce(total, group=mp_pg, op=dist.ReduceOp.MAX)
        if extra_reduce_group is not None and extra_reduce_group.size() > 1:
            dist.all_reduce(total, group=extra_reduce_group, op=dist.ReduceOp.MAX)
    else:
        if grads:
            norms = torch._foreach_norm(grads, norm_type)
            total = torch.stack([n.float() for n in norms]).pow(norm_type).sum()
        else:
            total = torch.zeros([], dtype=torch.float, device=device)
        dist.all_reduce(total, group=mp_pg, op=dist.ReduceOp.SUM)
        if extra_reduce_group is not None and extra_reduce_group.size() > 1:
            dist.all_reduce(total, group=extra_reduce_group, op=dist.ReduceOp.SUM)
        total = total.pow(1.0 / norm_type)
    clip_coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    if scale_slices is not None:
        targets = list(scale_slices)
    elif grad_slices is not None:
        targets = grads
    elif grad_accumulator is not None:
        targets = [grad_accumulator.get_grad_buffer(n) for n, _ in named_parameters]
    else:
        targets = [p.grad for _, p in named_parameters if p.grad is not None]
    if targets:
        # one fused multiply over all tensors, coefficient read on the device
        torch._foreach_mul_(targets, clip_coef.to(targets[0].dtype))
    return total
