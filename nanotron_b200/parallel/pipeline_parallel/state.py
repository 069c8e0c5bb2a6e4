"""Per-batch pipeline bookkeeping: which tensors crossed a stage boundary in each micro-batch, and the exchange of their
gradients (capability parity: reference src/nanotron/parallel/pipeline_parallel/state.py).

The design follows from the two one-directional lanes of ``p2p.py``:

* Nothing is queued.  An activation is sent the moment its ``PipelineBlock`` hands it over (asynchronously, never waited
  on by the computing stream) and received the moment the consuming block asks for it.
* A received activation that requires grad is an autograd *leaf*.  After the backward of its micro-batch its ``.grad`` is
  the gradient the producer stage needs, so no custom autograd function and no placeholder tensors are involved: the
  backward of a micro-batch is ONE ``torch.autograd.backward`` call whose roots are the local loss terms plus the
  activations this stage sent onwards, seeded with the gradients received for them.
* Gradients carry no header (shape and dtype are the activation's) and cross each boundary in the order the activations
  crossed it; both sides derive that order from the same per-micro-batch records, so it does not depend on the order in
  which autograd happens to visit nodes.  A received activation that took no part in the loss still gets a (zero)
  gradient sent back, which keeps the two sides matched instead of hanging.

Engines drive a state with ``begin_micro_batch`` / ``backward_micro_batch`` / ``finish``.
"""
from __future__ import annotations

import collections
import dataclasses
from abc import ABC, abstractmethod
from typing import Deque, List, Optional, Tuple

import torch

from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.pipeline_parallel.p2p import BWD, FWD, P2P

logger = get_logger(__name__)


@dataclasses.dataclass
class MicroBatchRecord:
    """What one micro-batch's forward left behind on this stage."""

    index: int
    roots: List[torch.Tensor] = dataclasses.field(default_factory=list)  # local scalars to differentiate (the loss)
    sent: List[Tuple[torch.Tensor, int, P2P]] = dataclasses.field(default_factory=list)  # (activation, to_rank, p2p), grad expected back
    received: List[Tuple[torch.Tensor, int, P2P]] = dataclasses.field(default_factory=list)  # (leaf, from_rank, p2p), grad owed


class PipelineBatchState(ABC):
    """What ``PipelineBlock`` needs from the schedule that is running."""

    @abstractmethod
    def send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P) -> None:
        ...

    @abstractmethod
    def recv_activation(self, from_rank: int, p2p: P2P) -> torch.Tensor:
        ...

    @abstractmethod
    def register_activation_requiring_backward(self, activation: torch.Tensor) -> None:
        ...


class PipelineTrainBatchState(PipelineBatchState):
    def __init__(self):
        self.pending: Deque[MicroBatchRecord] = collections.deque()  # forwarded, not yet backwarded (oldest first)
        self.current: Optional[MicroBatchRecord] = None
        self.nb_forwards = 0
        self.nb_backwards = 0
        self._p2ps: List[P2P] = []

    # ------------------------------------------------------------------ forward side
    def _note(self, p2p: P2P):
        if all(p is not p2p for p in self._p2ps):
            self._p2ps.append(p2p)
            p2p.begin_round()  # first use in this batch: it is at a micro-batch boundary (shapes learnt in earlier batches replay)

    def begin_micro_batch(self) -> MicroBatchRecord:
        for p in self._p2ps:
            p.begin_round()
        self.current = MicroBatchRecord(index=self.nb_forwards)
        self.pending.append(self.current)
        self.nb_forwards += 1
        return self.current

    def register_activation_requiring_backward(self, activation: torch.Tensor) -> None:
        self.current.roots.append(activation)

    def send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P) -> None:
        self._note(p2p)
        p2p.send(activation, to_rank, FWD)
        if activation.requires_grad and torch.is_grad_enabled():
            self.current.sent.append((activation, to_rank, p2p))

    def recv_activation(self, from_rank: int, p2p: P2P) -> torch.Tensor:
        self._note(p2p)
        ticket = p2p.recv(from_rank, FWD)
        wants_grad = ticket.requires_grad and torch.is_grad_enabled()
        ticket.requires_grad = wants_grad
        tensor = ticket.wait()
        if wants_grad:
            self.current.received.append((tensor, from_rank, p2p))
        return tensor

    # ------------------------------------------------------------------ backward side
    def backward_micro_batch(self, grad_accumulator=None) -> bool:
        """Backward of the oldest micro-batch still pending.  Returns False when there was nothing to differentiate."""
        if not self.pending:
            return False
        mb = self.pending.popleft()
        if self.current is mb:
            self.current = None
        # gradients of what went downstream, in the order it went
        tickets = [p2p.recv_like(act, to_rank, BWD) for act, to_rank, p2p in mb.sent]
        roots = list(mb.roots) + [act for act, _, _ in mb.sent]
        seeds = [None] * len(mb.roots) + [t.wait() for t in tickets]
        did = False
        if roots:
            if grad_accumulator is None:
                torch.autograd.backward(roots, seeds)
            else:
                grad_accumulator.backward(roots, seeds)
            did = True
        # gradients owed upstream, in the order the activations arrived
        for leaf, from_rank, p2p in mb.received:
            g = leaf.grad
            if g is None:
                g = torch.zeros_like(leaf)  # took no part in the loss: keep the exchange matched
            p2p.send_raw(g, from_rank, BWD)
            leaf.grad = None
        self.nb_backwards += 1
        return did

    def drop_pending(self):
        """Forward-only use (validation): forget the records, nothing will be differentiated."""
        self.pending.clear()
        self.current = None

    def finish(self):
        """End of the batch: every micro-batch was differentiated; retire the sends."""
        assert not self.pending, f"{len(self.pending)} micro-batches were forwarded but never backwarded"
        for p in self._p2ps:
            p.drain()

    # name kept for callers written against the reference engine
    check_buffers_empty = finish


class PipelineEvalBatchState(PipelineBatchState):
    """Inference (generation): activations only, exchanged eagerly and always with a header because shapes change from one
    decoding step to the next.  The last stage feeds the first one inside the decoding loop; sending at once is what
    keeps that cycle from waiting on itself."""

    def __init__(self):
        self._p2ps: List[P2P] = []

    def send_activation(self, activation: torch.Tensor, to_rank: int, p2p: P2P) -> None:
        p2p.send_tensors([activation], to_rank=to_rank, static=False)

    def recv_activation(self, from_rank: int, p2p: P2P) -> torch.Tensor:
        return p2p.recv_tensors(num_tensors=1, from_rank=from_rank, static=False)[0].requires_grad_(False)

    def register_activation_requiring_backward(self, activation: torch.Tensor) -> None:
        pass

    def begin_micro_batch(self):
        return None

    def finish(self):
        pass

    check_buffers_empty = finish
