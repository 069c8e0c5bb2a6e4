"""Small host-side helpers (parity: reference src/nanotron/utils.py)."""
from __future__ import annotations

import functools
import inspect
import os
import socket
from contextlib import ExitStack, contextmanager
from typing import Callable, ContextManager, List, Optional, Tuple

import torch
from torch import nn


class Singleton(type):
    """Metaclass that keeps one instance per class."""

    _instances: dict = {}

    def __call__(cls, *args, **kwargs):
        if cls not in cls._instances:
            cls._instances[cls] = super().__call__(*args, **kwargs)
        return cls._instances[cls]


class ContextManagers:
    """Enter a list of context managers as one."""

    def __init__(self, context_managers: List[ContextManager]):
        self.context_managers = context_managers
        self.stack = ExitStack()

    def __enter__(self):
        for cm in self.context_managers:
            self.stack.enter_context(cm)

    def __exit__(self, *args, **kwargs):
        self.stack.__exit__(*args, **kwargs)


_NVTX = {"usable": None}


@contextmanager
def annotate(name: str):
    """Name a region for the profilers: a ``torch.profiler`` record and, on a CUDA build, an NVTX range (visible in Nsight
    timelines beside the kernels launched inside).  A build without NVTX just loses the range."""
    if _NVTX["usable"] is None:
        _NVTX["usable"] = torch.cuda.is_available()
    pushed = False
    if _NVTX["usable"]:
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:
            _NVTX["usable"] = False
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


@contextmanager
def main_rank_first(group):
    """Rank 0 of ``group`` runs the body first, the others after it finished."""
    import nanotron_b200.distributed as dist

    is_main = dist.get_rank(group) == 0
    if is_main:
        yield
    dist.barrier(group)
    if not is_main:
        yield


@contextmanager
def local_ranks_zero_first(group=None):
    """The first rank of every node runs the body before the other ranks of that node."""
    import nanotron_b200.distributed as dist

    is_main = int(os.environ.get("LOCAL_RANK", "0")) == 0
    if is_main:
        yield
    dist.barrier(group)
    if not is_main:
        yield


def checkpoint_method(attr_name: str):
    """Decorator: recompute the method's activations in backward when ``self.<attr_name>`` is truthy."""

    def decorator(fn: Callable):
        @functools.wraps(fn)
        def wrapper(self, *args, **kwargs):
            if not getattr(self, attr_name):
                return fn(self, *args, **kwargs)
            sig = inspect.signature(fn)
            bound = sig.bind(self, *args, **kwargs)
            bound.apply_defaults()
            names = [n for n in bound.arguments if n != "self"]
            values = [bound.arguments[n] for n in names]

            def run(*flat):
                return fn(self, **dict(zip(names, flat)))

            from torch.utils.checkpoint import checkpoint

            return checkpoint(run, *values, use_reentrant=False)

        return wrapper

    return decorator


def get_parameter_and_parent_module(target: str, root_module: nn.Module) -> Tuple[nn.Parameter, nn.Module, str]:
    """Resolve ``a.b.c.weight`` to (parameter, module ``a.b.c``, ``"weight"``)."""
    module_path, _, param_name = target.rpartition(".")
    mod = root_module.get_submodule(module_path)
    if not hasattr(mod, param_name):
        raise AttributeError(f"{mod._get_name()} has no attribute `{param_name}`")
    param = getattr(mod, param_name)
    if not isinstance(param, nn.Parameter):
        raise AttributeError(f"`{param_name}` is not an nn.Parameter")
    return param, mod, param_name


def get_untyped_storage(tensor: torch.Tensor) -> torch.UntypedStorage:
    return tensor.untyped_storage()


def tensor_from_untyped_storage(untyped_storage: torch.UntypedStorage, dtype: torch.dtype) -> torch.Tensor:
    """View raw bytes as a 1-D tensor of ``dtype``."""
    t = torch.empty([], dtype=dtype, device=untyped_storage.device)
    t.set_(untyped_storage)
    return t


def find_free_port(min_port: int = 2000, max_port: int = 65000) -> int:
    import random

    for _ in range(1000):
        port = random.randint(min_port, max_port)
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", port))
                return port
            except OSError:
                continue
    raise RuntimeError("no free port found")


def assert_tensor_synced_across_pg(tensor: torch.Tensor, pg, msg: Optional[Callable[[str], str]] = None, reference_rank: int = 0):
    """Raise if ``tensor`` differs from the copy held by ``reference_rank`` of ``pg``."""
    import nanotron_b200.distributed as dist

    if dist.get_rank(pg) == reference_rank:
        ref = tensor.detach().clone()
    else:
        ref = torch.empty_like(tensor)
    dist.broadcast(ref, src=dist.get_global_rank(pg, reference_rank), group=pg)
    try:
        torch.testing.assert_close(tensor, ref, atol=0, rtol=0)
    except AssertionError as e:
        raise AssertionError(msg(str(e)) if msg else str(e))
