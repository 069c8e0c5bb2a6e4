"""Autograd-aware collectives used between tensor-parallel layers.

Parity: reference src/nanotron/parallel/tensor_parallel/distributed_differentiable_primitives.py:24-146.
Each forward collective pairs with its transpose in backward: identity<->all-reduce, all-gather<->reduce-scatter.
All of them act on dim 0 (the token dimension of the token-flat activation layout).
"""
from __future__ import annotations

from typing import Optional

import torch

import nanotron_b200.distributed as dist


class DifferentiableIdentity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, group: Optional[dist.ProcessGroup]):
        ctx.group = group
        return tensor

    @staticmethod
    def backward(ctx, grad_output):
        return DifferentiableAllReduceSum.apply(grad_output, ctx.group), None


class DifferentiableAllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, group: Optional[dist.ProcessGroup]):
        if group is None or group.size() == 1:
            return tensor
        tensor = tensor.contiguous().clone() if tensor.requires_grad or not tensor.is_contiguous() else tensor
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
        return tensor

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class DifferentiableAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, group: Optional[dist.ProcessGroup]):
        ctx.group = group
        if group is None or group.size() == 1:
            return tensor
        tensor = tensor.contiguous()
        out = torch.empty((tensor.shape[0] * group.size(), *tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
        dist.all_gather_into_tensor(out, tensor, group=group)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return DifferentiableReduceScatterSum.apply(grad_output, ctx.group), None


class DifferentiableReduceScatterSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, group: Optional[dist.ProcessGroup]):
        ctx.group = group
        if group is None or group.size() == 1:
            return tensor
        tensor = tensor.contiguous()
        assert tensor.shape[0] % group.size() == 0, f"dim 0 ({tensor.shape[0]}) must be divisible by the group size ({group.size()})"
        out = torch.empty((tensor.shape[0] // group.size(), *tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
        dist.reduce_scatter_tensor(out, tensor, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return DifferentiableAllGather.apply(grad_output, ctx.group), None


def differentiable_identity(tensor, group=None):
    return DifferentiableIdentity.apply(tensor, group)


def differentiable_all_reduce_sum(tensor, group=None):
    return DifferentiableAllReduceSum.apply(tensor, group)


def differentiable_all_gather(tensor, group=None):
    return DifferentiableAllGather.apply(tensor, group)


def differentiable_reduce_scatter_sum(tensor, group=None):
    return DifferentiableReduceScatterSum.apply(tensor, group)
