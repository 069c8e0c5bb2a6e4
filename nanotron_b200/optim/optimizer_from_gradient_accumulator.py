"""The link of the optimizer chain that swaps half-precision parameters for the fp32 master copies kept by a gradient
accumulator, and keeps the accumulator in step with the optimizer
(API parity: reference src/nanotron/optim/optimizer_from_gradient_accumulator.py).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Optional, Set, Tuple, Union

import torch

from nanotron_b200.optim.base import BaseOptimizer
from nanotron_b200.optim.gradient_accumulator import GradientAccumulator
from nanotron_b200.optim.inherit_from_other_optimizer import InheritFromOtherOptimizer

_KEY = "gradient_accumulator"


def _as_groups(named_params_or_groups) -> List[Dict[str, Any]]:
    """[(name, param), ...] or [{"named_params": [...], **options}, ...] -> the second form, with lists that can be read twice."""
    items = list(named_params_or_groups)
    if not items or not isinstance(items[0], dict):
        items = [{"named_params": items}]
    return [dict(group, named_params=list(group["named_params"])) for group in items]


class OptimizerFromGradientAccumulator(InheritFromOtherOptimizer):
    def __init__(
        self,
        gradient_accumulator_builder: Callable[[Iterable[Tuple[str, torch.Tensor]]], GradientAccumulator],
        named_params_or_groups: Iterable[Union[Tuple[str, torch.Tensor], Dict[str, Any]]],
        optimizer_builder: Callable[[Iterable[Dict[str, Any]]], BaseOptimizer],
    ):
        groups = _as_groups(named_params_or_groups)
        unique: Dict[str, torch.Tensor] = {}
        for group in groups:
            for name, param in group["named_params"]:
                if unique.setdefault(name, param) is not param:
                    raise AssertionError(f"duplicate parameter name {name}")
        self.gradient_accumulator = accumulator = gradient_accumulator_builder(unique.items())
        # the optimizer below works on the accumulator's fp32 masters
        for group in groups:
            group["named_params"] = [(name, accumulator.get_parameter_for_optimizer(name)) for name, _ in group["named_params"]]
        inner = optimizer_builder(groups)
        super().__init__(optimizer=inner, id_to_name=inner.id_to_name)

    def zero_grad(self):
        super().zero_grad()
        return self.gradient_accumulator.zero_grad()

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        loss = super().step(closure)
        self.gradient_accumulator.step()  # masters -> half-precision parameters
        return loss

    def state_dict_additional_keys(self) -> Set[str]:
        return super().state_dict_additional_keys() | {_KEY}

    def state_dict(self) -> dict:
        state = super().state_dict()
        assert _KEY not in state
        state[_KEY] = self.gradient_accumulator.state_dict()
        return state

    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        rest = {k: v for k, v in state_dict.items() if k != _KEY}
        super().load_state_dict(rest, map_location=map_location)
        self.gradient_accumulator.load_state_dict(state_dict[_KEY])
