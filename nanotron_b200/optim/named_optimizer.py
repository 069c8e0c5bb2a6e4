"""Optimizer that remembers parameter names (parity: reference src/nanotron/optim/named_optimizer.py)."""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, Optional, Tuple, Union

import torch

from nanotron_b200.optim.inherit_from_other_optimizer import InheritFromOtherOptimizer


class NamedOptimizer(InheritFromOtherOptimizer):
    def __init__(
        self,
        named_params_or_groups: Iterable[Union[Tuple[str, torch.Tensor], Dict[str, Any]]],
        optimizer_builder: Callable[[Iterable[Dict[str, Any]]], torch.optim.Optimizer],
    ):
        named_param_groups = list(named_params_or_groups)
        if len(named_param_groups) == 0 or not isinstance(named_param_groups[0], dict):
            named_param_groups = [{"named_params": named_param_groups}]
        id_to_name = {}
        params = []
        for group in named_param_groups:
            assert "named_params" in group, f"param_groups must contain a 'named_params' key, got a dict with keys {group.keys()}"
            group = dict(group)
            group["named_params"] = list(group["named_params"])
            for name, param in group["named_params"]:
                id_to_name[id(param)] = name
            params.append({**{k: v for k, v in group.items() if k != "named_params"}, "params": [p for _, p in group["named_params"]]})
        name_to_id = {v: k for k, v in id_to_name.items()}
        assert len(id_to_name) == len(name_to_id), "several parameters share a name"
        for g in params:
            assert len(g["params"]) > 0 or len(params) > 1, "Specified named_params is empty"
        params = [g for g in params if len(g["params"]) > 0] or params
        super().__init__(optimizer=optimizer_builder(params), id_to_name=id_to_name)

    def state_dict(self) -> dict:
        sd = super().state_dict()
        assert "names" not in sd
        index_to_name = {}
        idx = 0
        for group in self.optimizer.param_groups:
            for p in group["params"]:
                index_to_name[idx] = self.id_to_name[id(p)]
                idx += 1
        sd["names"] = index_to_name
        return sd

    def load_state_dict(self, state_dict: dict, map_location: Optional[Union[str, torch.device]] = None) -> None:
        state_dict = dict(state_dict)
        names = state_dict.pop("names", None)
        if names is not None:
            idx = 0
            for group in self.optimizer.param_groups:
                for p in group["params"]:
                    saved = names.get(idx, names.get(str(idx)))
                    assert saved == self.id_to_name[id(p)], f"optimizer state name mismatch at index {idx}: {saved} vs {self.id_to_name[id(p)]}"
                    idx += 1
        return super().load_state_dict(state_dict, map_location=map_location)
