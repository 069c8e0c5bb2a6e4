"""Per-batch bookkeeping of pipeline communication (parity: reference src/nanotron/parallel/pipeline_parallel/state.py).

Sends and receives requested by ``PipelineBlock`` during a forward/backward are queued here and executed by
``run_communication`` in a fixed order (send activations, recv activations, send grads, recv grads), which is
what keeps every pair of neighbouring stages matched.
"""
from __future__ import annotations

import collections
import dataclasses
from abc import ABC, abstractmethod
from typing import List

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P

logger = get_logger(__name__)


@dataclasses.dataclass
class SendActivation:
    activation: torch.Tensor
    to_rank: int
    p2p: P2P

    def __call__(self):
        self.p2p.send_tensors([self.activation], to_rank=self.to_rank)


@dataclasses.dataclass
class RecvActivation:
    from_rank: int
    p2p: P2P

    def __call__(self) -> torch.Tensor:
        return self.p2p.recv_tensors(num_tensors=1, from_rank=self.from_rank)[0]


@dataclasses.dataclass
class SendGrad:
    grad: torch.Tensor
    to_rank: int
    p2p: P2P

    def __call__(self):
        self.p2p.send_tensors([self.grad], to_rank=self.to_rank)


@dataclasses.dataclass
class RecvGrad:
    from_rank: int
    p2p: P2P

    def __call__(self) -> torch.Tensor:
        return self.p2p.recv_tensors(num_tensors=1, from_rank=self.from_rank)[0]


class PipelineBatchState(ABC):
    activations_buffer = collections.deque()

    @abstractmethod
    def register_activation_requiring_backward(self, activation: torch.Tensor):
        ...

    @abstractmethod
    def register_send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P):
        ...

    @abstractmethod
    def register_recv_activation(self, from_rank: int, p2p: P2P):
        ...

    @abstractmethod
    def register_send_grad(self, grad: torch.Tensor, to_rank: int, p2p: P2P):
        ...

    @abstractmethod
    def register_recv_grad(self, from_rank: int, p2p: P2P):
        ...

    @abstractmethod
    def run_communication(self, send_only_activation: bool = False):
        ...

    @abstractmethod
    def new_micro_batch_forward(self):
        ...

    @abstractmethod
    def pop_last_activations_requiring_backward(self) -> List[torch.Tensor]:
        ...


@dataclasses.dataclass
class PipelineTrainBatchState(PipelineBatchState):
    microbatches_activations_to_send = collections.deque()
    microbatches_activations_to_recv = collections.deque()
    microbatches_grads_to_send = collections.deque()
    microbatches_grads_to_recv = collections.deque()
    grads_buffer = collections.deque()
    activations_buffer = collections.deque()
    microbatches_activations_requiring_backward = collections.deque()
    nb_backwards: int = 0
    nb_forwards: int = 0

    def __post_init__(self):
        # dataclass class-level deques would be shared between instances: give each instance its own
        self.microbatches_activations_to_send = collections.deque()
        self.microbatches_activations_to_recv = collections.deque()
        self.microbatches_grads_to_send = collections.deque()
        self.microbatches_grads_to_recv = collections.deque()
        self.grads_buffer = collections.deque()
        self.activations_buffer = collections.deque()
        self.microbatches_activations_requiring_backward = collections.deque()

    def new_micro_batch_forward(self):
        self.microbatches_activations_requiring_backward.append(collections.deque())

    def register_activation_requiring_backward(self, activation: torch.Tensor):
        self.microbatches_activations_requiring_backward[-1].append(activation)

    def register_send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P):
        self.microbatches_activations_to_send.append(SendActivation(activation=activation, to_rank=to_rank, p2p=p2p))

    def register_recv_activation(self, from_rank: int, p2p: P2P):
        self.microbatches_activations_to_recv.append(RecvActivation(from_rank=from_rank, p2p=p2p))

    def register_send_grad(self, grad: torch.Tensor, to_rank: int, p2p: P2P):
        self.microbatches_grads_to_send.append(SendGrad(grad=grad, to_rank=to_rank, p2p=p2p))

    def register_recv_grad(self, from_rank: int, p2p: P2P):
        self.microbatches_grads_to_recv.append(RecvGrad(from_rank=from_rank, p2p=p2p))

    def run_communication(self, send_only_activation: bool = False):
        """Drain the queues.  ``send_only_activation``: used at the end of a forward when peers are not yet ready
        to exchange gradients."""
        logger.debug(
            f"run_communication: act_send={len(self.microbatches_activations_to_send)} act_recv={len(self.microbatches_activations_to_recv)} "
            f"grad_send={len(self.microbatches_grads_to_send)} grad_recv={len(self.microbatches_grads_to_recv)}"
        )
        while len(self.microbatches_activations_to_send) > 0:
            self.microbatches_activations_to_send.popleft()()
        if send_only_activation:
            return
        while len(self.microbatches_activations_to_recv) > 0:
            self.activations_buffer.append(self.microbatches_activations_to_recv.popleft()())
        while len(self.microbatches_grads_to_send) > 0:
            self.microbatches_grads_to_send.popleft()()
        while len(self.microbatches_grads_to_recv) > 0:
            self.grads_buffer.append(self.microbatches_grads_to_recv.popleft()())

    def pop_last_activations_requiring_backward(self) -> List[torch.Tensor]:
        return self.microbatches_activations_requiring_backward.popleft()

    def check_buffers_empty(self):
        assert len(self.microbatches_activations_requiring_backward) == 0, f"There are still activations that require backward: {len(self.microbatches_activations_requiring_backward)}"
        assert len(self.microbatches_activations_to_send) == 0, "There are activations left for me to send still"
        assert len(self.microbatches_activations_to_recv) == 0, "There are activations left for me to recv still"
        assert len(self.microbatches_grads_to_send) == 0, "There are gradients left for me to send still"
        assert len(self.microbatches_grads_to_recv) == 0, "There are gradients left for me to recv still"


@dataclasses.dataclass
class PipelineEvalBatchState(PipelineBatchState):
    """Inference: only activations travel, nothing is kept for backward."""

    microbatches_activations_to_send = collections.deque()
    microbatches_activations_to_recv = collections.deque()
    activations_buffer = collections.deque()

    def __post_init__(self):
        self.microbatches_activations_to_send = collections.deque()
        self.microbatches_activations_to_recv = collections.deque()
        self.activations_buffer = collections.deque()

    def new_micro_batch_forward(self):
        pass

    def register_activation_requiring_backward(self, activation: torch.Tensor):
        pass

    def register_send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P):
        self.microbatches_activations_to_send.append(SendActivation(activation=activation, to_rank=to_rank, p2p=p2p))
        # sending eagerly avoids a cyclic wait when the last stage feeds the first one (decoding loop)
        self.microbatches_activations_to_send.popleft()()

    def register_recv_activation(self, from_rank: int, p2p: P2P):
        self.microbatches_activations_to_recv.append(RecvActivation(from_rank=from_rank, p2p=p2p))
        self.activations_buffer.append(self.microbatches_activations_to_recv.popleft()())

    def register_send_grad(self, grad: torch.Tensor, to_rank: int, p2p: P2P):
        raise NotImplementedError("You can't register a send grad in pipeline eval mode")

    def register_recv_grad(self, from_rank: int, p2p: P2P):
        raise NotImplementedError("You can't register a recv grad in pipeline eval mode")

    def run_communication(self, send_only_activation: bool = False):
        while len(self.microbatches_activations_to_send) > 0:
            self.microbatches_activations_to_send.popleft()()
        while len(self.microbatches_activations_to_recv) > 0:
            self.activations_buffer.append(self.microbatches_activations_to_recv.popleft()())

    def pop_last_activations_requiring_backward(self) -> List[torch.Tensor]:
        return []

    def check_buffers_empty(self):
        assert len(self.microbatches_activations_to_send) == 0
        assert len(self.microbatches_activations_to_recv) == 0
        assert len(self.activations_buffer) == 0
