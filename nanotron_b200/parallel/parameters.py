"""``NanotronParameter``: an ``nn.Parameter`` carrying sharding / tying metadata.

Parity: reference src/nanotron/parallel/parameters.py:16-202.  The metadata drives checkpoint naming,
gradient synchronisation of tied parameters, and topology-agnostic checkpoint loading.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn


@dataclasses.dataclass
class SlicesPair:
    """One contiguous block of a sharded tensor: where it sits locally and where it sits in the unsharded tensor."""

    local_slices: Tuple[slice, ...]
    global_slices: Tuple[slice, ...]

    @staticmethod
    def slice_to_str(s: slice) -> str:
        return f"{s.start},{s.stop},{s.step}"

    @staticmethod
    def str_to_slice(s: str) -> slice:
        return slice(*(int(x) if x != "None" else None for x in s.split(",")))

    def __str__(self) -> str:
        local = "|".join(map(self.slice_to_str, self.local_slices))
        glob = "|".join(map(self.slice_to_str, self.global_slices))
        return f"local_slices:{local}#global_slices:{glob}"

    @classmethod
    def from_str(cls, string: str) -> "SlicesPair":
        local_part, global_part = string.split("#")
        lp, ls = local_part.split(":")
        gp, gs = global_part.split(":")
        assert lp == "local_slices" and gp == "global_slices", string
        return cls(
            local_slices=tuple(map(cls.str_to_slice, ls.split("|"))),
            global_slices=tuple(map(cls.str_to_slice, gs.split("|"))),
        )

    @classmethod
    def tuple_to_str(cls, pairs: Tuple["SlicesPair", ...]) -> str:
        return ";".join(map(str, pairs))

    @classmethod
    def tuple_from_str(cls, string: str) -> Tuple["SlicesPair", ...]:
        return tuple(map(cls.from_str, string.split(";")))


@dataclasses.dataclass
class TiedInfo:
    name: str
    root_module: nn.Module  # `name` is relative to this module
    global_ranks: Tuple[int, ...]
    reduce_op: Optional[Any]  # dist.ReduceOp or None (no gradient reduction needed)

    def get_full_name_from_model(self, model: nn.Module) -> str:
        if self.root_module is model:
            return self.name
        for prefix, mod in model.named_modules():
            if mod is self.root_module:
                return f"{prefix}.{self.name}" if prefix else self.name
        raise ValueError(f"root module of tied parameter `{self.name}` is not inside the given model")

    def get_full_name_from_module_id_to_prefix(self, module_id_to_prefix: Dict[int, str]) -> str:
        return f"{module_id_to_prefix[id(self.root_module)]}{self.name}"


@dataclasses.dataclass
class ShardedInfo:
    global_ranks: Tuple[int, ...]
    local_global_slices_pairs: Tuple[SlicesPair, ...]
    unsharded_shape: Tuple[int, ...]

    def is_tp_sharded(self, parallel_context) -> bool:
        return set(self.global_ranks) == set(_group_ranks(parallel_context.tp_pg))

    def is_expert_sharded(self, parallel_context) -> bool:
        return parallel_context.expert_parallel_size > 1 and set(self.global_ranks) == set(_group_ranks(parallel_context.ep_pg))

    def is_dp_sharded(self, parallel_context) -> bool:
        return set(self.global_ranks) == set(_group_ranks(parallel_context.dp_pg))


def _group_ranks(pg):
    import nanotron_b200.distributed as dist

    return dist.get_global_ranks(pg)


class NanotronParameter(nn.Parameter):
    NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME = "__nanotron_metadata__"
    NANOTRON_PARAMETER_METADATA_TIED_KEY = "tied"
    NANOTRON_PARAMETER_METADATA_SHARDED_KEY = "sharded"

    def __new__(cls, tensor: torch.Tensor, requires_grad: bool = True):
        param = nn.Parameter._make_subclass(cls, tensor.detach(), requires_grad)
        if isinstance(tensor, NanotronParameter):
            meta = dict(getattr(tensor, cls.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME))
        else:
            meta = {}
        setattr(param, cls.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME, meta)
        return param

    def __deepcopy__(self, memo):
        out = NanotronParameter(self.data.clone(memory_format=torch.preserve_format), self.requires_grad)
        setattr(out, self.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME, dict(self._meta))
        memo[id(self)] = out
        return out

    @property
    def _meta(self) -> Dict[str, Any]:
        if not hasattr(self, self.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME):
            setattr(self, self.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME, {})
        return getattr(self, self.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME)

    def _set_metadata(self, key: str, value: Any):
        if key in self._meta:
            raise ValueError(f"We shouldn't override previous metadata. Key to be overridden: {key}, current metadata: {self._meta}")
        self._meta[key] = value

    def mark_as_tied(self, name: str, global_ranks: Tuple[int, ...], reduce_op, root_module: nn.Module):
        self._set_metadata(
            self.NANOTRON_PARAMETER_METADATA_TIED_KEY,
            TiedInfo(name=name, global_ranks=tuple(global_ranks), reduce_op=reduce_op, root_module=root_module),
        )

    def get_tied_info(self) -> TiedInfo:
        return self._meta[self.NANOTRON_PARAMETER_METADATA_TIED_KEY]

    @property
    def is_tied(self) -> bool:
        return self.NANOTRON_PARAMETER_METADATA_TIED_KEY in self._meta

    def mark_as_sharded(self, global_ranks: Tuple[int, ...], local_global_slices_pairs: Tuple[SlicesPair, ...], unsharded_shape: Tuple[int, ...]):
        self._set_metadata(
            self.NANOTRON_PARAMETER_METADATA_SHARDED_KEY,
            ShardedInfo(global_ranks=tuple(global_ranks), local_global_slices_pairs=tuple(local_global_slices_pairs), unsharded_shape=tuple(unsharded_shape)),
        )

    def get_sharded_info(self) -> ShardedInfo:
        return self._meta[self.NANOTRON_PARAMETER_METADATA_SHARDED_KEY]

    @property
    def is_sharded(self) -> bool:
        return self.NANOTRON_PARAMETER_METADATA_SHARDED_KEY in self._meta


def sanity_check(root_module: nn.Module):
    """Every parameter of a nanotron model must be a NanotronParameter."""
    for name, param in root_module.named_parameters():
        if not isinstance(param, NanotronParameter):
            raise ValueError(f"Nanotronrequires model to be in Nanotron format, ie all parameters are required to be a NanotronParameter. {name} isn't.")
