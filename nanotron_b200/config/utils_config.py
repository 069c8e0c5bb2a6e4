"""Enums, (de)serialisation of dataclass trees to plain YAML-able values, and a strict dataclass loader.

The loader replaces the third-party ``dacite`` dependency of the reference
(reference src/nanotron/config/config.py:609-648): unknown keys are errors, ``Union`` fields are resolved
by trying each member in order, and registered type hooks convert strings to enums / dtypes / engines.
"""
from __future__ import annotations

import dataclasses
import typing
from dataclasses import fields, is_dataclass
from enum import Enum, auto
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Type, Union

import torch


class RecomputeGranularity(Enum):
    SELECTIVE = auto()
    FULL = auto()


class InitScalingMethod(Enum):
    NONE = auto()
    NUM_LAYERS = auto()
    LAYER_INDEX = auto()
    MODEL_SCALE = auto()


class SamplerType(Enum):
    TOP_P = auto()
    TOP_K = auto()
    GREEDY = auto()
    BASIC = auto()


_STR_TO_DTYPE = {
    "float32": torch.float32,
    "float64": torch.float64,
    "complex64": torch.complex64,
    "complex128": torch.complex128,
    "float16": torch.float16,
    "bfloat16": torch.bfloat16,
    "uint8": torch.uint8,
    "int8": torch.int8,
    "int16": torch.int16,
    "int32": torch.int32,
    "int64": torch.int64,
    "bool": torch.bool,
    "float8_e4m3fn": torch.float8_e4m3fn,
    "float8_e5m2": torch.float8_e5m2,
}
_DTYPE_TO_STR = {v: k for k, v in _STR_TO_DTYPE.items()}


def cast_str_to_torch_dtype(str_dtype):
    if isinstance(str_dtype, torch.dtype):
        return str_dtype
    if str_dtype in _STR_TO_DTYPE:
        return _STR_TO_DTYPE[str_dtype]
    raise ValueError(f"unknown dtype {str_dtype}")


def cast_str_to_pipeline_engine(str_pp_engine):
    from nanotron_b200.parallel.pipeline_parallel.engine import (
        AllForwardAllBackwardPipelineEngine,
        OneForwardOneBackwardPipelineEngine,
        PipelineEngine,
    )

    if isinstance(str_pp_engine, PipelineEngine):
        return str_pp_engine
    if str_pp_engine == "afab":
        return AllForwardAllBackwardPipelineEngine()
    if str_pp_engine == "1f1b":
        return OneForwardOneBackwardPipelineEngine()
    raise ValueError(f"pp_engine should be a string selected in ['afab', '1f1b'] and not {str_pp_engine}")


def serialize(data) -> Any:
    """Dataclass tree -> nested dict/list of YAML scalars. ``None`` passes through."""
    if data is None:
        return None
    if not is_dataclass(data):
        return _serialize_value(data)
    out = {}
    for f in fields(data):
        out[f.name] = _serialize_value(getattr(data, f.name))
    return out


def _serialize_value(value):
    from nanotron_b200.parallel.pipeline_parallel.engine import (
        AllForwardAllBackwardPipelineEngine,
        OneForwardOneBackwardPipelineEngine,
        PipelineEngine,
    )
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode

    if is_dataclass(value) and not isinstance(value, type):
        return serialize(value)
    if isinstance(value, Path):
        return str(value)
    if isinstance(value, PipelineEngine):
        if isinstance(value, OneForwardOneBackwardPipelineEngine):
            return "1f1b"
        if isinstance(value, AllForwardAllBackwardPipelineEngine):
            return "afab"
        raise ValueError(f"unknown pipeline engine {value}")
    if isinstance(value, TensorParallelLinearMode):
        return value.name
    if isinstance(value, (RecomputeGranularity, InitScalingMethod, SamplerType)):
        return value.name
    if isinstance(value, Enum):
        return value.name
    if isinstance(value, torch.dtype):
        return _DTYPE_TO_STR[value]
    if isinstance(value, (list, tuple)):
        return [_serialize_value(v) for v in value]
    if isinstance(value, dict):
        return {k: _serialize_value(v) for k, v in value.items()}
    return value


# --------------------------------------------------------------------------- strict loader
class ConfigError(ValueError):
    pass


def _default_type_hooks() -> Dict[Any, Callable]:
    from nanotron_b200.parallel.pipeline_parallel.engine import PipelineEngine
    from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode

    return {
        torch.dtype: cast_str_to_torch_dtype,
        PipelineEngine: cast_str_to_pipeline_engine,
        TensorParallelLinearMode: lambda x: x if isinstance(x, TensorParallelLinearMode) else TensorParallelLinearMode[x.upper()],
        RecomputeGranularity: lambda x: x if isinstance(x, RecomputeGranularity) else RecomputeGranularity[x.upper()],
        InitScalingMethod: lambda x: x if isinstance(x, InitScalingMethod) else InitScalingMethod[x.upper()],
        SamplerType: lambda x: x if isinstance(x, SamplerType) else SamplerType[x.upper()],
        Path: lambda x: Path(x),
    }


def from_dict(data_class: Type, data: dict, strict: bool = True, type_hooks: Optional[Dict[Any, Callable]] = None, path: str = ""):
    """Build ``data_class`` from a plain dict, recursively."""
    hooks = _default_type_hooks()
    if type_hooks:
        hooks.update(type_hooks)
    return _build_dataclass(data_class, data, strict, hooks, path)


def _build_dataclass(cls, data, strict, hooks, path):
    if not isinstance(data, dict):
        raise ConfigError(f"{path or cls.__name__}: expected a mapping for {cls.__name__}, got {type(data).__name__}")
    hints = typing.get_type_hints(cls)
    known = {f.name: f for f in fields(cls)}
    if strict:
        extra = set(data) - set(known)
        if extra:
            raise ConfigError(f"{path or cls.__name__}: unknown keys {sorted(extra)} for {cls.__name__}")
    kwargs, post = {}, {}
    for name, f in known.items():
        if name in data:
            value = _convert(hints.get(name, Any), data[name], strict, hooks, f"{path}.{name}" if path else name)
            if f.init:
                kwargs[name] = value
            else:
                post[name] = value
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING and f.init:
            raise ConfigError(f"{path or cls.__name__}: missing required key `{name}` for {cls.__name__}")
    try:
        obj = cls(**kwargs)
    except TypeError as e:
        raise ConfigError(f"{path or cls.__name__}: {e}")
    for k, v in post.items():
        setattr(obj, k, v)
    return obj


def _convert(tp, value, strict, hooks, path):
    if tp is Any or tp is None:
        return value
    origin = typing.get_origin(tp)
    if origin is Union:
        args = typing.get_args(tp)
        if value is None and type(None) in args:
            return None
        errors = []
        # exact-type matches first so that e.g. str is not coerced to a list member
        for a in args:
            if a is type(None):
                continue
            try:
                return _convert(a, value, strict, hooks, path)
            except (ConfigError, ValueError, TypeError, KeyError, AssertionError) as e:
                errors.append(f"{getattr(a, '__name__', a)}: {e}")
        raise ConfigError(f"{path}: value {value!r} matches no member of {tp}: " + " | ".join(errors))
    if tp in hooks:
        return hooks[tp](value)
    if is_dataclass(tp):
        if isinstance(value, tp):
            return value
        return _build_dataclass(tp, value, strict, hooks, path)
    if origin in (list, typing.List):
        (inner,) = typing.get_args(tp) or (Any,)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list, got {type(value).__name__}")
        return [_convert(inner, v, strict, hooks, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (tuple, typing.Tuple):
        inner = typing.get_args(tp)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a sequence")
        if len(inner) == 2 and inner[1] is Ellipsis:
            return tuple(_convert(inner[0], v, strict, hooks, path) for v in value)
        return tuple(_convert(t, v, strict, hooks, path) for t, v in zip(inner, value))
    if origin in (dict, typing.Dict):
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping")
        return value
    if origin is typing.Literal:
        if value not in typing.get_args(tp):
            raise ConfigError(f"{path}: {value!r} not in {typing.get_args(tp)}")
        return value
    if isinstance(tp, type):
        if issubclass(tp, Enum):
            return value if isinstance(value, tp) else tp[str(value).upper()]
        if tp is float and isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if tp is float and isinstance(value, str):
            return float(value)  # yaml reads 1e-5 without a dot as str
        if tp is int and isinstance(value, bool):
            raise ConfigError(f"{path}: expected int, got bool")
        if tp is bool and not isinstance(value, bool):
            raise ConfigError(f"{path}: expected bool, got {type(value).__name__}")
        if isinstance(value, tp):
            return value
        raise ConfigError(f"{path}: expected {tp.__name__}, got {type(value).__name__} ({value!r})")
    return value
