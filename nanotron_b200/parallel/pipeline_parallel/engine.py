"""Pipeline schedules: all-forward-all-backward and one-forward-one-backward.

Parity: reference src/nanotron/parallel/pipeline_parallel/engine.py:24-348.  A model wrapper may expose
``no_sync()`` (context manager that suppresses gradient synchronisation) and ``trigger_grad_sync()``; the engine
enters ``no_sync`` for every micro-batch but the last so data-parallel reduction happens once per step and can
overlap the last backward.
"""
from __future__ import annotations

import contextlib
from abc import ABC, abstractmethod
from typing import Dict, Iterable, List, Optional, Union

import torch
from torch import nn as torch_nn

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.pipeline_parallel.context_manager import attach_pipeline_state_to_model
from nanotron_b200.parallel.pipeline_parallel.state import PipelineEvalBatchState, PipelineTrainBatchState
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer
from nanotron_b200.utils import ContextManagers

logger = get_logger(__name__)


class PipelineEngine(ABC):
    def __init__(self):
        self.nb_microbatches: Optional[int] = None

    def __eq__(self, other):
        return type(self) is type(other)

    def __hash__(self):
        return hash(type(self).__name__)

    def forward(self, context: ContextManagers, state: PipelineTrainBatchState, micro_batch: Dict[str, Union[torch.Tensor, TensorPointer]], model: torch_nn.Module):
        state.new_micro_batch_forward()
        with context:
            output = model(**micro_batch)
        if not isinstance(output, dict):
            output = {"loss": output}
        for k, v in output.items():
            if not isinstance(v, TensorPointer):
                output[k] = v / self.nb_microbatches
        # the loss tensor is what backward starts from on the last stage
        if not isinstance(output["loss"], TensorPointer):
            assert output["loss"].requires_grad or not torch.is_grad_enabled()
            state.register_activation_requiring_backward(output["loss"])
        return output

    @staticmethod
    def _get_fwd_context(model: torch_nn.Module):
        return ContextManagers([])

    def backward(self, context: ContextManagers, state: PipelineTrainBatchState, grad_accumulator=None):
        if len(state.microbatches_activations_requiring_backward) == 0:
            return
        with context:
            activations = state.pop_last_activations_requiring_backward()
            if len(activations) == 0:
                return
            if grad_accumulator is None:
                sum(activations).backward()
            else:
                grad_accumulator.backward(sum(activations))
        # tensors sent in forward that turned out unused raise here rather than hang
        state.nb_backwards += 1

    def _get_bwd_context(self, model: torch_nn.Module, nb_backwards: int, grad_accumulator=None):
        is_last = nb_backwards == self.nb_microbatches - 1
        cms = []
        if hasattr(model, "no_sync") and not is_last:
            cms.append(model.no_sync())
        elif is_last and hasattr(model, "prepare_last_backward"):
            cms.append(model.prepare_last_backward())
        return ContextManagers(cms)

    @abstractmethod
    def train_batch_iter(self, model: torch_nn.Module, pg: dist.ProcessGroup, batch: Iterable[Dict[str, Union[torch.Tensor, TensorPointer]]], nb_microbatches: int, grad_accumulator=None) -> Iterable[Dict[str, Union[torch.Tensor, TensorPointer]]]:
        ...

    @torch.inference_mode()
    def validate_batch_iter(self, model: torch_nn.Module, batch: Iterable[Dict[str, Union[torch.Tensor, TensorPointer]]], nb_microbatches: int) -> Iterable[Dict[str, Union[torch.Tensor, TensorPointer]]]:
        state = PipelineTrainBatchState()
        self.nb_microbatches = nb_microbatches
        outputs = []
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for micro_batch in batch:
                context = self._get_fwd_context(model=model)
                output = self.forward(context=context, state=state, micro_batch=micro_batch, model=model)
                for _ in range(len(state.microbatches_activations_to_send)):
                    state.microbatches_activations_to_send.popleft()()
                if not isinstance(output, dict):
                    output = {"loss": output}
                if not isinstance(output["loss"], TensorPointer):
                    output = {k: v.detach() for k, v in output.items()}
                outputs.append(output)
                # nothing is backpropagated in validation
                state.microbatches_activations_requiring_backward.clear()
        return outputs


class AllForwardAllBackwardPipelineEngine(PipelineEngine):
    def train_batch_iter(self, model, pg, batch, nb_microbatches, grad_accumulator=None):
        state = PipelineTrainBatchState()
        self.nb_microbatches = nb_microbatches
        outputs = []
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for micro_batch in batch:
                context = self._get_fwd_context(model=model)
                output = self.forward(context=context, state=state, micro_batch=micro_batch, model=model)
                # send what this stage produced right away so the next stage can start
                for _ in range(len(state.microbatches_activations_to_send)):
                    state.microbatches_activations_to_send.popleft()()
                if not isinstance(output["loss"], TensorPointer):
                    output = {k: v.detach() for k, v in output.items()}
                outputs.append(output)
            for _ in range(len(state.microbatches_activations_requiring_backward)):
                context = self._get_bwd_context(model=model, nb_backwards=state.nb_backwards, grad_accumulator=grad_accumulator)
                self.backward(context=context, state=state, grad_accumulator=grad_accumulator)
                for _ in range(len(state.microbatches_grads_to_send)):
                    state.microbatches_grads_to_send.popleft()()
            state.check_buffers_empty()
        return outputs


class OneForwardOneBackwardPipelineEngine(PipelineEngine):
    def train_batch_iter(self, model, pg, batch, nb_microbatches, grad_accumulator=None):
        """Warm-up of ``pp_size - rank - 1`` forwards, then alternate one forward / one backward, then drain."""
        self.nb_microbatches = nb_microbatches
        assert self.nb_microbatches >= pg.size() - 1, f"Number of microbatches ({self.nb_microbatches}) must be at least PP_SIZE-1={pg.size() - 1} when using the OneForwardOneBackwardPipelineEngine"
        state = PipelineTrainBatchState()
        outputs = []
        batch = iter(batch)
        current_pp_rank = dist.get_rank(pg)
        with attach_pipeline_state_to_model(model=model, pipeline_state=state):
            for _ in range(pg.size() - current_pp_rank - 1):
                micro_batch = next(batch)
                context = self._get_fwd_context(model=model)
                output = self.forward(context=context, state=state, micro_batch=micro_batch, model=model)
                for _ in range(len(state.microbatches_activations_to_send)):
                    state.microbatches_activations_to_send.popleft()()
                if not isinstance(output["loss"], TensorPointer):
                    output = {k: v.detach() for k, v in output.items()}
                outputs.append(output)
            for micro_batch in batch:
                context = self._get_fwd_context(model=model)
                output = self.forward(context=context, state=state, micro_batch=micro_batch, model=model)
                # only activations: the next stage may not be ready to hand gradients back yet
                state.run_communication(send_only_activation=True)
                if not isinstance(output["loss"], TensorPointer):
                    output = {k: v.detach() for k, v in output.items()}
                outputs.append(output)
                context = self._get_bwd_context(model=model, nb_backwards=state.nb_backwards, grad_accumulator=grad_accumulator)
                self.backward(context=context, state=state, grad_accumulator=grad_accumulator)
            state.run_communication()
            assert len(state.microbatches_activations_to_send) == 0
            # cool-down: remaining backwards
            for _ in range(len(state.microbatches_activations_requiring_backward)):
                context = self._get_bwd_context(model=model, nb_backwards=state.nb_backwards, grad_accumulator=grad_accumulator)
                self.backward(context=context, state=state, grad_accumulator=grad_accumulator)
                for _ in range(len(state.microbatches_grads_to_send)):
                    state.microbatches_grads_to_send.popleft()()
            state.check_buffers_empty()
        return outputs
