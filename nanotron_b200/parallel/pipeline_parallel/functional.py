"""Autograd glue that lets activations cross pipeline stages (parity: reference
src/nanotron/parallel/pipeline_parallel/functional.py:9-119)."""
from __future__ import annotations

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
from nanotron_b200.parallel.pipeline_parallel.state import PipelineBatchState

logger = get_logger(__name__)


class SendTensorToPipelineBuffer(torch.autograd.Function):
    """Queue ``activation`` for sending.  Returns a zero-size-cost scalar that requires grad: calling backward on
    it receives the activation's gradient from the next stage and continues backpropagation locally."""

    @staticmethod
    def forward(ctx, activation: torch.Tensor, to_rank: int, p2p: P2P, pipeline_state: PipelineBatchState):
        assert activation.requires_grad
        ctx.p2p, ctx.to_rank, ctx.pipeline_state = p2p, to_rank, pipeline_state
        pipeline_state.register_send_activation(activation, to_rank=to_rank, p2p=p2p)
        return torch.tensor(1, dtype=torch.float, device="cpu", requires_grad=True)

    @staticmethod
    def backward(ctx, grad_tensor):
        state = ctx.pipeline_state
        state.register_recv_grad(from_rank=ctx.to_rank, p2p=ctx.p2p)
        if len(state.grads_buffer) == 0:
            state.run_communication()
        return state.grads_buffer.popleft(), None, None, None


class SendTensorWithoutGradientToPipelineBuffer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dummy_input: torch.Tensor, activation: torch.Tensor, to_rank: int, p2p: P2P, pipeline_state: PipelineBatchState):
        assert dummy_input.requires_grad
        assert activation.requires_grad is False
        pipeline_state.register_send_activation(activation, to_rank=to_rank, p2p=p2p)
        return torch.tensor(1, dtype=torch.float, device="cpu", requires_grad=True)

    @staticmethod
    def backward(ctx, grad_tensor):
        return torch.tensor(1, dtype=torch.float, device="cpu"), None, None, None, None


def send_to_pipeline_state_buffer(tensor: torch.Tensor, to_rank: int, p2p: P2P, pipeline_state: PipelineBatchState):
    if tensor.requires_grad:
        result = SendTensorToPipelineBuffer.apply(tensor, to_rank, p2p, pipeline_state)
        pipeline_state.register_activation_requiring_backward(result)
    else:
        # nothing to backpropagate: queue a plain send
        pipeline_state.register_send_activation(tensor, to_rank=to_rank, p2p=p2p)


class RecvTensorFromPipelineBuffer(torch.autograd.Function):
    """Take the next received activation; its backward queues the gradient to be sent to the producer stage."""

    @staticmethod
    def forward(ctx, activation: torch.Tensor, from_rank: int, p2p: P2P, pipeline_state: PipelineBatchState):
        ctx.pipeline_state, ctx.p2p, ctx.from_rank = pipeline_state, p2p, from_rank
        return activation

    @staticmethod
    def backward(ctx, grad_tensor):
        ctx.pipeline_state.register_send_grad(grad_tensor, to_rank=ctx.from_rank, p2p=ctx.p2p)
        return None, None, None, None


def recv_from_pipeline_state_buffer(from_rank: int, p2p: P2P, pipeline_state: PipelineBatchState):
    pipeline_state.register_recv_activation(from_rank=from_rank, p2p=p2p)
    if len(pipeline_state.activations_buffer) == 0:
        pipeline_state.run_communication()
    activation = pipeline_state.activations_buffer.popleft()
    if activation.requires_grad:
        return RecvTensorFromPipelineBuffer.apply(activation, from_rank, p2p, pipeline_state)
    return activation
