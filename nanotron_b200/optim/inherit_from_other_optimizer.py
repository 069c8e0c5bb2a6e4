"""Optimizer wrappers form a chain (ZeRO -> gradient-accumulator optimizer -> named optimizer -> torch optimizer); this is the
link: everything a wrapper does not define itself is answered by the optimizer it wraps
(API parity: reference src/nanotron/optim/inherit_from_other_optimizer.py).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterator, Optional, Set, Union

import torch

from nanotron_b200.optim.base import BaseOptimizer, custom_load_state_dict


def _passes_on(name: str):
    """A method that hands the call to the wrapped optimizer unchanged."""

    def method(self, *args, **kwargs):
        return getattr(self.optimizer, name)(*args, **kwargs)

    method.__name__ = name
    method.__qualname__ = f"InheritFromOtherOptimizer.{name}"
    return method


class InheritFromOtherOptimizer(BaseOptimizer):
    # the parts of the optimizer protocol that a plain link forwards as they are
    zero_grad = _passes_on("zero_grad")
    state_dict = _passes_on("state_dict")
    __getstate__ = _passes_on("__getstate__")
    __setstate__ = _passes_on("__setstate__")

    def __init__(self, optimizer, id_to_name: Dict[int, str]):
        self.id_to_name = id_to_name
        if isinstance(optimizer, torch.optim.Optimizer):
            # end of the chain: give this torch optimizer (this instance only) a loader that understands map_location
            def load(state_dict, map_location=None, _inner=optimizer):
                return custom_load_state_dict(_inner, state_dict, map_location=map_location)

            optimizer.load_state_dict = load
        self.optimizer = optimizer

    def links(self) -> Iterator[object]:
        """This wrapper, the one it wraps, ... down to the torch optimizer."""
        node = self
        while node is not None:
            yield node
            node = None if isinstance(node, torch.optim.Optimizer) else getattr(node, "optimizer", None)

    def __repr__(self):
        return " -> ".join(type(link).__name__ for link in self.links())

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        return self.optimizer.load_state_dict(state_dict, map_location=map_location)

    def step(self, closure: Optional[Callable[[], float]] = None) -> Optional[float]:
        return self.optimizer.step() if closure is None else self.optimizer.step(closure=closure)

    def state_dict_additional_keys(self) -> Set[str]:
        """Keys that wrappers further down add to the torch optimizer's state dict; a wrapper that adds one extends this."""
        inner = self.optimizer
        return inner.state_dict_additional_keys() if isinstance(inner, InheritFromOtherOptimizer) else set()

    def get_base_optimizer(self):
        *_, last = self.links()
        return last

    def inherit_from(self, cls) -> bool:
        return any(isinstance(link, cls) for link in self.links())
