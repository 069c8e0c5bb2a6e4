"""Optimizer stepping the fp32 master weights held by a gradient accumulator (parity: reference
src/nanotron/optim/optimizer_from_gradient_accumulator.py)."""
from __future__ import annotations

from functools import cache
from typing import Any, Callable, Dict, Iterable, Optional, Set, Tuple, Union

import torch

from nanotron_b200.optim.base import BaseOptimizer
from nanotron_b200.optim.gradient_accumulator import GradientAccumulator
from nanotron_b200.optim.inherit_from_other_optimizer import InheritFromOtherOptimizer


class OptimizerFromGradientAccumulator(InheritFromOtherOptimizer):
    def __init__(
        self,
        gradient_accumulator_builder: Callable[[Iterable[Tuple[str, torch.Tensor]]], GradientAccumulator],
        named_params_or_groups: Iterable[Union[Tuple[str, torch.Tensor], Dict[str, Any]]],
        optimizer_builder: Callable[[Iterable[Dict[str, Any]]], BaseOptimizer],
    ):
        groups = list(named_params_or_groups)
        if len(groups) == 0 or not isinstance(groups[0], dict):
            groups = [{"named_params": groups}]
        groups = [{**g, "named_params": list(g["named_params"])} for g in groups]
        name_to_param = {}
        for g in groups:
            for name, param in g["named_params"]:
                assert name not in name_to_param or name_to_param[name] is param, f"duplicate parameter name {name}"
                name_to_param[name] = param
        gradient_accumulator = gradient_accumulator_builder(name_to_param.items())
        self.gradient_accumulator = gradient_accumulator
        # the inner optimizer sees the fp32 master copies instead of the half-precision parameters
        converted = [
            {**{k: v for k, v in g.items() if k != "named_params"}, "named_params": [(n, gradient_accumulator.get_parameter_for_optimizer(n)) for n, _ in g["named_params"]]}
            for g in groups
        ]
        optimizer = optimizer_builder(converted)
        super().__init__(optimizer=optimizer, id_to_name=optimizer.id_to_name)

    def zero_grad(self):
        super().zero_grad()
        return self.gradient_accumulator.zero_grad()

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        loss = super().step(closure)
        self.gradient_accumulator.step()
        return loss

    @cache
    def state_dict_additional_keys(self) -> Set[str]:
        return super().state_dict_additional_keys() | {"gradient_accumulator"}

    def state_dict(self) -> dict:
        sd = super().state_dict()
        assert "gradient_accumulator" not in sd
        sd["gradient_accumulator"] = self.gradient_accumulator.state_dict()
        return sd

    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        state_dict = dict(state_dict)
        ga = state_dict.pop("gradient_accumulator")
        super().load_state_dict(state_dict, map_location=map_location)
        self.gradient_accumulator.load_state_dict(ga)
