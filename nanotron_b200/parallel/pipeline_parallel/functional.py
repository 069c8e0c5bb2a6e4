"""How a tensor crosses a pipeline-stage boundary during a schedule (same entry points as the reference's
src/nanotron/parallel/pipeline_parallel/functional.py:9-119, different mechanism).

The reference wraps both ends in autograd functions: the sender gets back a CPU scalar that stands for "the rest of the
network" and whose backward receives the gradient, the receiver's function queues the gradient for sending.  Here the
received activation is simply a leaf of the local autograd graph and the sent one a root of the local backward; the
pipeline state (``state.py``) seeds and collects their gradients around a single ``torch.autograd.backward`` call, so
these two helpers only forward to the state.
"""
from __future__ import annotations

import torch

from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
from nanotron_b200.parallel.pipeline_parallel.state import PipelineBatchState


def send_to_pipeline_state_buffer(tensor: torch.Tensor, to_rank: int, p2p: P2P, pipeline_state: PipelineBatchState) -> None:
    """Hand ``tensor`` to pipeline rank ``to_rank``.  If it requires grad, its gradient comes back during the backward of the
    same micro-batch and backpropagation continues from it."""
    pipeline_state.send_activation(tensor, to_rank=to_rank, p2p=p2p)


def recv_from_pipeline_state_buffer(from_rank: int, p2p: P2P, pipeline_state: PipelineBatchState) -> torch.Tensor:
    """Next tensor from pipeline rank ``from_rank``; when the sender marked it as requiring grad it is returned as a leaf whose
    gradient the state sends back after the micro-batch's backward."""
    return pipeline_state.recv_activation(from_rank=from_rank, p2p=p2p)
