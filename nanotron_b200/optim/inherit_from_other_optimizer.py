"""Delegating optimizer wrapper (parity: reference src/nanotron/optim/inherit_from_other_optimizer.py)."""
from __future__ import annotations

from functools import cache
from typing import Callable, Dict, Optional, Set, Union

import torch

from nanotron_b200.optim.base import BaseOptimizer, custom_load_state_dict


class InheritFromOtherOptimizer(BaseOptimizer):
    def __init__(self, optimizer, id_to_name: Dict[int, str]):
        self.id_to_name = id_to_name
        if isinstance(optimizer, torch.optim.Optimizer):
            # bind the map_location-aware loader to this instance only
            optimizer.load_state_dict = lambda sd, map_location=None, _o=optimizer: custom_load_state_dict(_o, sd, map_location=map_location)
        self.optimizer = optimizer

    def __getstate__(self):
        return self.optimizer.__getstate__()

    def __setstate__(self, state):
        return self.optimizer.__setstate__(state)

    def __repr__(self):
        return f"{self.__class__.__name__}({repr(self.optimizer)})"

    def zero_grad(self):
        return self.optimizer.zero_grad()

    @cache
    def state_dict_additional_keys(self) -> Set[str]:
        if isinstance(self.optimizer, InheritFromOtherOptimizer):
            return self.optimizer.state_dict_additional_keys()
        return set()

    def state_dict(self) -> dict:
        return self.optimizer.state_dict()

    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        return self.optimizer.load_state_dict(state_dict, map_location=map_location)

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        return self.optimizer.step(closure=closure) if closure is not None else self.optimizer.step()

    def get_base_optimizer(self):
        if isinstance(self.optimizer, torch.optim.Optimizer):
            return self.optimizer
        return self.optimizer.get_base_optimizer()

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def inherit_from(self, cls):
        if isinstance(self, cls):
            return True
        if isinstance(self.optimizer, InheritFromOtherOptimizer):
            return self.optimizer.inherit_from(cls)
        return isinstance(self.optimizer, cls)
