"""Model base class and pipeline-aware construction (parity: reference src/nanotron/models/base.py:24-344)."""
from __future__ import annotations

import threading
from abc import ABCMeta, abstractmethod
from contextlib import contextmanager
from typing import TYPE_CHECKING, Callable, Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import LoggingCollectorMixin, get_logger, log_rank
from nanotron_b200.parallel.context import ParallelContext
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

if TYPE_CHECKING:
    from nanotron_b200.config import NanotronConfigs
    from nanotron_b200.parallel.parameters import NanotronParameter

logger = get_logger(__name__)
_init_state = threading.local()


class NanotronModel(nn.Module, LoggingCollectorMixin, metaclass=ABCMeta):
    """Base of every trainable model.  Subclasses hold ``parallel_context``, ``config`` and ``parallel_config``."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.parallel_context: ParallelContext
        self.config: "NanotronConfigs"
        self.module_id_to_prefix: Dict[int, str]
        # attributes of sub-modules are not copied when a model is wrapped
        self.input_pp_rank: int
        self.output_pp_rank: int
        self.init_model_randomly: Callable

    def get_named_params_with_correct_tied(self) -> Iterator[Tuple[str, "NanotronParameter"]]:
        """Named parameters where a tied parameter is reported under its canonical (tie) name."""

        def params_gen():
            for name, param in self.named_parameters():
                if getattr(param, "is_tied", False):
                    yield (param.get_tied_info().get_full_name_from_module_id_to_prefix(module_id_to_prefix=self.module_id_to_prefix), param)
                else:
                    yield name, param

        yield from params_gen()

    @abstractmethod
    def init_model_randomly(self, config):
        ...

    def tie_custom_params(self) -> None:
        """Hook for models that tie extra parameters (e.g. multi-query kv projections)."""
        return

    def get_embeddings_lm_head_tied_names(self) -> List[str]:
        """Names of the embedding and lm_head weights when they are to be tied; [] otherwise."""
        return []

    def get_named_params_without_weight_decay(self) -> List[str]:
        return []

    def before_tbi_sanity_checks(self) -> None:
        pass

    def after_tbi_sanity_checks(self) -> None:
        pass

    def before_optim_step_sanity_checks(self) -> None:
        pass

    def after_optim_step_sanity_checks(self) -> None:
        pass

    def log_modules(self, level: int = 10, group: Optional[dist.ProcessGroup] = None, rank: int = 0):
        for name, module in self.named_modules():
            if not isinstance(module, PipelineBlock):
                continue
            log_rank(f"module_name: {name} | PP: {module.rank}/{self.parallel_context.pp_pg.size()}", logger=logger, level=level, group=group, rank=rank)

    @property
    def named_modules_in_pp_rank(self) -> Dict[str, nn.Module]:
        """Leaf-most modules (those holding parameters directly) living on this pipeline rank."""

        def has_direct_params(m: nn.Module) -> bool:
            return any(True for _ in m.parameters(recurse=False))

        return {name: m for name, m in self.named_modules() if has_direct_params(m)}


class DTypeInvariantTensor(torch.Tensor):
    """Tensor that refuses dtype conversion (used for fp32-only buffers such as rotary frequencies)."""

    def __new__(cls, *args, **kwargs):
        return super().__new__(cls, *args, **kwargs)

    def detach(self, *args, **kwargs):
        raise RuntimeError("Cannot detach an DTypeInvariantTensor")

    def to(self, *args, **kwargs):
        if "dtype" in kwargs or any(isinstance(arg, torch.dtype) for arg in args):
            raise RuntimeError("Cannot change the type of an DTypeInvariantTensor")
        return super().to(*args, **kwargs)

    def type(self, *args, **kwargs):
        raise RuntimeError("Cannot change the type of an DTypeInvariantTensor")

    def float(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to float")

    def double(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to double")

    def half(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to half")

    def long(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to long")

    def int(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to int")

    def bool(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to boolean")

    def bfloat16(self, *args, **kwargs):
        raise RuntimeError("Cannot convert the type of an DTypeInvariantTensor to bfloat16")


def build_model(
    model_builder: Callable[[], NanotronModel],
    parallel_context: ParallelContext,
    dtype: torch.dtype,
    target_pp_ranks: Optional[List[int]] = None,
    device: Optional[torch.device] = None,
) -> NanotronModel:
    """Instantiate the model skeleton on every rank and materialise each ``PipelineBlock`` on its stage.

    Stage assignment balances ``model.get_block_compute_costs()`` (cost per block class): block i goes to the stage
    whose cumulative-cost threshold it falls under, so stages carry about equal compute.  ``target_pp_ranks``
    overrides the assignment block by block."""
    if device is None:
        device = parallel_context.device
    model: NanotronModel = model_builder()
    model.input_pp_rank = 0
    model.output_pp_rank = parallel_context.pp_pg.size() - 1
    blocks = [m for m in model.modules() if isinstance(m, PipelineBlock)]
    with init_on_device_and_dtype(device=device, dtype=dtype):
        if target_pp_ranks is not None:
            assert len(target_pp_ranks) == len(blocks)
            for block, rank in zip(blocks, target_pp_ranks):
                block.build_and_set_rank(rank)
        else:
            pp_size = parallel_context.pp_pg.size()
            costs_table = model.get_block_compute_costs() if hasattr(model, "get_block_compute_costs") else {}
            costs = [costs_table.get(b.module_builder, 0) for b in blocks]
            cum = np.cumsum(costs)
            total = cum[-1] if len(cum) else 0
            thresholds = [total * (r + 1) / pp_size for r in range(pp_size)]
            rank = 0
            for block, c in zip(blocks, cum):
                assert rank < pp_size
                block.build_and_set_rank(rank)
                if rank != pp_size - 1 and c > thresholds[rank]:
                    rank += 1
    model.module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in model.named_modules()}
    model.module_id_to_prefix[id(model)] = ""
    return model


def ignore_init_on_device_and_dtype(func):
    """Decorator: parameters created inside keep the dtype/device they ask for (e.g. an fp32 router weight)."""

    def wrapper(*args, **kwargs):
        old = getattr(_init_state, "ignore", False)
        _init_state.ignore = True
        try:
            return func(*args, **kwargs)
        finally:
            _init_state.ignore = old

    return wrapper


@contextmanager
def init_on_device_and_dtype(device: torch.device = torch.device("cpu"), dtype: torch.dtype = torch.float):
    """Inside the block, every newly registered parameter / buffer is created on ``device``; floating-point
    parameters take ``dtype``.  Tensor factory functions default to that device too, so modules never allocate
    on the host first.  ``DTypeInvariantTensor`` buffers keep their dtype."""
    old_register_parameter = nn.Module.register_parameter
    old_register_buffer = nn.Module.register_buffer

    def _move(t, keep_dtype=False):
        if keep_dtype or not t.is_floating_point():
            return t.to(device)
        return t.to(device=device, dtype=dtype)

    def register_parameter(module, name, param):
        old_register_parameter(module, name, param)
        if param is None or getattr(_init_state, "ignore", False):
            if param is not None:
                p = module._parameters[name]
                module._parameters[name] = type(p)(p.data.to(device), requires_grad=p.requires_grad) if p.device != device else p
            return
        p = module._parameters[name]
        new_data = _move(p.data)
        if new_data is not p.data:
            cls = type(p)
            kwargs = {"requires_grad": p.requires_grad}
            module._parameters[name] = cls(new_data, **kwargs)
            if hasattr(p, "__nanotron_metadata__"):
                module._parameters[name].__nanotron_metadata__ = p.__nanotron_metadata__

    def register_buffer(module, name, buffer, persistent=True):
        old_register_buffer(module, name, buffer, persistent=persistent)
        if buffer is not None:
            if isinstance(buffer, DTypeInvariantTensor) or getattr(_init_state, "ignore", False):
                module._buffers[name] = buffer.to(device)
            else:
                module._buffers[name] = _move(buffer, keep_dtype=True)

    factories = ["empty", "zeros", "ones", "full", "arange", "randn", "rand"]
    old_factories = {n: getattr(torch, n) for n in factories}

    def patch(fn):
        def wrapper(*args, **kwargs):
            if kwargs.get("device") is None:
                kwargs["device"] = device
            return fn(*args, **kwargs)

        return wrapper

    try:
        nn.Module.register_parameter = register_parameter
        nn.Module.register_buffer = register_buffer
        for n, f in old_factories.items():
            setattr(torch, n, patch(f))
        yield
    finally:
        nn.Module.register_parameter = old_register_parameter
        nn.Module.register_buffer = old_register_buffer
        for n, f in old_factories.items():
            setattr(torch, n, f)


def check_model_has_grad(model: NanotronModel, parallel_context: ParallelContext):
    """At least one parameter of every pipeline stage must require grad (otherwise the schedule would hang)."""
    for stage in range(parallel_context.pp_pg.size()):
        if dist.get_rank(parallel_context.pp_pg) != stage:
            continue
        if not any(p.requires_grad for p in model.parameters()):
            raise ValueError(
                f"pipeline stage {stage} of {parallel_context.pp_pg.size()} holds no trainable parameter: the model has too few blocks "
                f"(or too uneven block costs) for this many stages; use fewer pipeline stages"
            )
