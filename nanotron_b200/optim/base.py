"""Optimizer interface and a ``load_state_dict`` that honours ``map_location`` (parity: reference src/nanotron/optim/base.py)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from collections import defaultdict
from copy import deepcopy
from itertools import chain
from typing import Any, Callable, Dict, List, Optional, Set, Union

import torch


class BaseOptimizer(ABC):
    id_to_name: Dict[int, str]
    param_groups: List[Dict[str, Any]]

    @abstractmethod
    def __getstate__(self):
        ...

    @abstractmethod
    def __setstate__(self, state):
        ...

    @abstractmethod
    def __repr__(self):
        ...

    @abstractmethod
    def zero_grad(self):
        ...

    @abstractmethod
    def state_dict_additional_keys(self) -> Set[str]:
        """Keys of the optimizer state dict that do not live inside the per-parameter ``state``."""

    @abstractmethod
    def state_dict(self) -> dict:
        ...

    @abstractmethod
    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        ...

    @abstractmethod
    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        ...

    def inherit_from(self, cls) -> bool:
        ...


def custom_load_state_dict(self: torch.optim.Optimizer, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
    """``torch.optim.Optimizer.load_state_dict`` that places state tensors on ``map_location`` (default: the
    parameter's device) so a large state can be loaded on CPU first and moved right before the first step."""
    state_dict = deepcopy(state_dict) if map_location is None else state_dict
    groups = self.param_groups
    saved_groups = state_dict["param_groups"]
    if len(groups) != len(saved_groups):
        raise ValueError("loaded state dict has a different number of parameter groups")
    if any(len(g["params"]) != len(s["params"]) for g, s in zip(groups, saved_groups)):
        raise ValueError("loaded state dict contains a parameter group that doesn't match the size of optimizer's group")
    id_map = dict(zip(chain.from_iterable(g["params"] for g in saved_groups), chain.from_iterable(g["params"] for g in groups)))

    def cast(param, value, key=None):
        if isinstance(value, torch.Tensor):
            target = map_location if map_location is not None else param.device
            if key == "step":
                return value.to(dtype=torch.float32, device=target) if value.dim() == 0 and not getattr(self, "_step_on_device", False) else value.to(target)
            if param.is_floating_point() and value.is_floating_point():
                return value.to(dtype=param.dtype if value.dtype != torch.float32 else torch.float32, device=target)
            return value.to(device=target)
        if isinstance(value, dict):
            return {k: cast(param, v, key=k) for k, v in value.items()}
        return value

    state = defaultdict(dict)
    for k, v in state_dict["state"].items():
        if k in id_map:
            state[id_map[k]] = cast(id_map[k], v)
        else:
            state[k] = v

    def update_group(group, new_group):
        new_group["params"] = group["params"]
        return new_group

    self.__setstate__({"state": state, "param_groups": [update_group(g, ng) for g, ng in zip(groups, saved_groups)]})
