"""Minimal stand-in for the third-party ``dacite`` package (not installable offline), sufficient for the way the
reference uses it: ``from_dict(data_class, data, config=Config(cast=[...], type_hooks={...}, strict=True))``."""
from __future__ import annotations

import dataclasses
import typing
from dataclasses import dataclass, field, fields, is_dataclass
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Type, Union


class DaciteError(Exception):
    pass


class WrongTypeError(DaciteError):
    pass


class MissingValueError(DaciteError):
    pass


class UnexpectedDataError(DaciteError):
    pass


@dataclass
class Config:
    type_hooks: Dict[Any, Callable] = field(default_factory=dict)
    cast: List[Type] = field(default_factory=list)
    forward_references: Optional[Dict[str, Any]] = None
    check_types: bool = True
    strict: bool = False
    strict_unions_match: bool = False


def from_dict(data_class, data, config: Optional[Config] = None):
    config = config or Config()
    return _build(data_class, data, config)


def _build(cls, data, config):
    if not isinstance(data, dict):
        raise WrongTypeError(f"expected mapping for {cls.__name__}, got {type(data).__name__}")
    try:
        hints = typing.get_type_hints(cls, localns=config.forward_references)
    except Exception:
        hints = {f.name: f.type for f in fields(cls)}
    known = {f.name: f for f in fields(cls)}
    if config.strict:
        extra = set(data) - set(known)
        if extra:
            raise UnexpectedDataError(f"can not match {sorted(extra)} to any data class field of {cls.__name__}")
    kwargs, post = {}, {}
    for name, f in known.items():
        if name in data:
            v = _convert(hints.get(name, Any), data[name], config)
            (kwargs if f.init else post)[name] = v
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING and f.init:
            raise MissingValueError(f"missing value for field {name} of {cls.__name__}")
    obj = cls(**kwargs)
    for k, v in post.items():
        setattr(obj, k, v)
    return obj


def _convert(tp, value, config):
    if tp in config.type_hooks:
        return config.type_hooks[tp](value)
    if tp is Any:
        return value
    origin = typing.get_origin(tp)
    if origin is Union:
        args = typing.get_args(tp)
        if value is None and type(None) in args:
            return None
        last = None
        for a in args:
            if a is type(None):
                continue
            try:
                out = _convert(a, value, config)
                if is_dataclass(a) or a in config.type_hooks or _is_instance(out, a):
                    return out
            except Exception as e:  # try the next member
                last = e
        if last is not None and not any(_is_instance(value, a) for a in args if a is not type(None)):
            raise WrongTypeError(f"value {value!r} matches no member of {tp}: {last}")
        return value
    if is_dataclass(tp) and isinstance(tp, type):
        if isinstance(value, tp):
            return value
        return _build(tp, value, config)
    if origin in (list, typing.List):
        (inner,) = typing.get_args(tp) or (Any,)
        return [_convert(inner, v, config) for v in value]
    if origin in (tuple, typing.Tuple):
        inner = typing.get_args(tp)
        if len(inner) == 2 and inner[1] is Ellipsis:
            return tuple(_convert(inner[0], v, config) for v in value)
        return tuple(_convert(t, v, config) for t, v in zip(inner, value))
    if origin in (dict, typing.Dict):
        args = typing.get_args(tp)
        if len(args) == 2 and isinstance(value, dict):
            return {k: _convert(args[1], v, config) for k, v in value.items()}
        return value
    if isinstance(tp, type):
        for c in config.cast:
            if isinstance(c, type) and issubclass(tp, c) and not isinstance(value, tp):
                return tp(value)
        if issubclass(tp, Enum) and not isinstance(value, tp):
            raise WrongTypeError(f"{value!r} is not a {tp.__name__}")
        if tp is float and isinstance(value, int) and not isinstance(value, bool):
            return value
    return value


def _is_instance(value, tp) -> bool:
    origin = typing.get_origin(tp)
    if origin is not None:
        tp = origin
    try:
        return isinstance(value, tp)
    except TypeError:
        return True
