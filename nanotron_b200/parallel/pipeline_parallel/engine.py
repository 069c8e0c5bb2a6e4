"""Pipeline schedules: all-forward-all-backward (AFAB) and one-forward-one-backward (1F1B).

Capability parity: reference src/nanotron/parallel/pipeline_parallel/engine.py:24-348 (same class names and
``train_batch_iter`` / ``validate_batch_iter`` entry points).  A schedule here is only an order of ``forward`` and
``backward`` calls: communication needs no scheduling of its own because activations and gradients travel on separate
one-directional lanes and are sent the moment they exist (``p2p.py``, ``state.py``).

Data-parallel hooks: if the model (or the gradient accumulator) exposes ``no_sync()`` it is entered for every backward but the
last, and ``prepare_last_backward()`` (a context manager) wraps the last one, which is where gradient reduction that
overlaps the backward pass is armed.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, Iterable, List, Optional, Union

import torch
from torch import nn as torch_nn

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.pipeline_parallel.context_manager import attach_pipeline_state_to_model
from nanotron_b200.parallel.pipeline_parallel.state import PipelineTrainBatchState
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer
from nanotron_b200.utils import ContextManagers, annotate

logger = get_logger(__name__)
MicroBatch = Dict[str, Union[torch.Tensor, TensorPointer]]


class PipelineEngine(ABC):
    def __init__(self):
        self.nb_microbatches: Optional[int] = None

    def __eq__(self, other):
        return type(self) is type(other)

    def __hash__(self):
        return hash(type(self).__name__)

    # ------------------------------------------------------------------ one micro-batch
    def forward(self, context: ContextManagers, state: PipelineTrainBatchState, micro_batch: MicroBatch, model: torch_nn.Module) -> Dict:
        state.begin_micro_batch()
        with context:
            output = model(**micro_batch)
        if not isinstance(output, dict):
            output = {"loss": output}
        # every micro-batch contributes 1 / nb_microbatches of the step's loss (and of its gradient)
        output = {k: (v if isinstance(v, TensorPointer) else v / self.nb_microbatches) for k, v in output.items()}
        loss = output["loss"]
        if not isinstance(loss, TensorPointer):
            assert loss.requires_grad or not torch.is_grad_enabled()
            if loss.requires_grad:
                state.register_activation_requiring_backward(loss)
        return output

    @staticmethod
    def _get_fwd_context(model: torch_nn.Module):
        return ContextManagers([])

    def _get_bwd_context(self, model: torch_nn.Module, nb_backwards: int, grad_accumulator=None):
        last = nb_backwards == self.nb_microbatches - 1
        managers = []
        for owner in (model, grad_accumulator):
            if owner is None:
                continue
            if not last and hasattr(owner, "no_sync"):
                managers.append(owner.no_sync())
            elif last and hasattr(owner, "prepare_last_backward"):
                managers.append(owner.prepare_last_backward())
        return ContextManagers(managers)

    def backward(self, context: ContextManagers, state: PipelineTrainBatchState, grad_accumulator=None):
        with context:
            state.backward_micro_batch(grad_accumulator=grad_accumulator)

    def _one_forward(self, model, state, micro_batch, outputs: List[Dict]):
        with annotate("micro_batch_forward"):
            output = self.forward(context=self._get_fwd_context(model=model), state=state, micro_batch=micro_batch, model=model)
        if not isinstance(output["loss"], TensorPointer):
            output = {k: v.detach() for k, v in output.items()}
        outputs.append(output)

    def _one_backward(self, model, state, grad_accumulator):
        context = self._get_bwd_context(model=model, nb_backwards=state.nb_backwards, grad_accumulator=grad_accumulator)
        with annotate("micro_batch_backward"):
            self.backward(context=context, state=state, grad_accumulator=grad_accumulator)

    # ------------------------------------------------------------------ whole batches
    @abstractmethod
    def train_batch_iter(self, model: torch_nn.Module, pg: dist.ProcessGroup, batch: Iterable[MicroBatch], nb_microbatches: int, grad_accumulator=None) -> Iterable[Dict]:
        ...

    @torch.inference_mode()
    def validate_batch_iter(self, model: torch_nn.Module, batch: Iterable[MicroBatch], nb_microbatches: int) -> Iterable[Dict]:
        state = PipelineTrainBatchState()
        self.nb_microbatches = nb_microbatches
        outputs: List[Dict] = []
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for micro_batch in batch:
                self._one_forward(model, state, micro_batch, outputs)
            state.drop_pending()
            state.finish()
        return outputs


class AllForwardAllBackwardPipelineEngine(PipelineEngine):
    def train_batch_iter(self, model, pg, batch, nb_microbatches, grad_accumulator=None):
        self.nb_microbatches = nb_microbatches
        state = PipelineTrainBatchState()
        outputs: List[Dict] = []
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for micro_batch in batch:
                self._one_forward(model, state, micro_batch, outputs)
            for _ in range(len(outputs)):
                self._one_backward(model, state, grad_accumulator)
            state.finish()
        return outputs


class OneForwardOneBackwardPipelineEngine(PipelineEngine):
    def train_batch_iter(self, model, pg, batch, nb_microbatches, grad_accumulator=None):
        """Stage r of p runs ``p - r - 1`` forwards ahead (so the last stage alternates from the start), then one forward and one
        backward per remaining micro-batch, then the backwards it still owes.  At most ``p - r`` micro-batches of activations are
        alive on a stage, against all of them under AFAB."""
        self.nb_microbatches = nb_microbatches
        stages, me = pg.size(), dist.get_rank(pg)
        assert nb_microbatches >= stages - 1, f"Number of microbatches ({nb_microbatches}) must be at least PP_SIZE-1={stages - 1} when using the OneForwardOneBackwardPipelineEngine"
        ahead = min(stages - me - 1, nb_microbatches)
        state = PipelineTrainBatchState()
        outputs: List[Dict] = []
        feed = iter(batch)
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for _ in range(ahead):
                self._one_forward(model, state, next(feed), outputs)
            for micro_batch in feed:
                self._one_forward(model, state, micro_batch, outputs)
                self._one_backward(model, state, grad_accumulator)
            for _ in range(ahead):
                self._one_backward(model, state, grad_accumulator)
            state.finish()
        return outputs
