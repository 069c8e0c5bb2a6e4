"""Named timers backed by CUDA events or the host clock (parity: reference src/nanotron/logging/timers.py).

CUDA timers record events on the current stream and only synchronise the *last* end event when the
elapsed time is read, so timing a region does not stall the device.  On a CPU-only process every timer
falls back to ``time.perf_counter``.
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from enum import Enum
from functools import wraps
from typing import Callable, Dict, List, Optional

import torch


class TimerType(Enum):
    CPU = "cpu"
    CUDA = "cuda"


@dataclass
class TimerRecord:
    name: str
    timer_type: TimerType = TimerType.CUDA
    cuda_sync: bool = False
    enabled: bool = True
    _starts: List = field(default_factory=list)
    _ends: List = field(default_factory=list)
    _running: bool = False
    call_count: int = 0

    def __post_init__(self):
        if self.timer_type == TimerType.CUDA and not torch.cuda.is_available():
            self.timer_type = TimerType.CPU

    def start(self) -> "TimerRecord":
        if not self.enabled:
            return self
        if self._running:
            self.end()
        if self.timer_type == TimerType.CUDA:
            if self.cuda_sync:
                torch.cuda.synchronize()
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._starts.append(ev)
        else:
            self._starts.append(time.perf_counter())
        self._running = True
        return self

    def end(self) -> None:
        if not self.enabled or not self._running:
            return
        if self.timer_type == TimerType.CUDA:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._ends.append(ev)
            if self.cuda_sync:
                torch.cuda.synchronize()
        else:
            self._ends.append(time.perf_counter())
        self._running = False
        self.call_count += 1

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.end()

    def reset(self) -> None:
        self._starts.clear()
        self._ends.clear()
        self._running = False
        self.call_count = 0

    @property
    def elapsed(self) -> float:
        """Seconds of the most recent interval."""
        if not self._ends:
            return 0.0
        if self.timer_type == TimerType.CUDA:
            self._ends[-1].synchronize()
            return self._starts[len(self._ends) - 1].elapsed_time(self._ends[-1]) / 1000.0
        return self._ends[-1] - self._starts[len(self._ends) - 1]

    @property
    def total_time(self) -> float:
        if not self._ends:
            return 0.0
        if self.timer_type == TimerType.CUDA:
            self._ends[-1].synchronize()
            return sum(s.elapsed_time(e) for s, e in zip(self._starts, self._ends)) / 1000.0
        return sum(e - s for s, e in zip(self._starts, self._ends))

    @property
    def average_time(self) -> float:
        return self.total_time / self.call_count if self.call_count else 0.0


class Timers:
    """Registry of :class:`TimerRecord`; usable as ``timers("name")`` context manager or decorator."""

    def __init__(self):
        self._timers: Dict[str, TimerRecord] = {}
        self._enabled = os.environ.get("ENABLE_TIMERS", "0") == "1"
        self._default_type = TimerType.CUDA
        self._default_sync = False

    def enable(self):
        self._enabled = True

    def disable(self):
        self._enabled = False

    def is_enabled(self) -> bool:
        return self._enabled

    def configure(self, timer_type: TimerType = TimerType.CUDA, cuda_sync: bool = False, enabled: Optional[bool] = None):
        self._default_type = timer_type
        self._default_sync = cuda_sync
        if enabled is not None:
            self._enabled = enabled

    def __call__(self, name=None, timer_type=None, cuda_sync: Optional[bool] = None, enabled: Optional[bool] = None):
        if callable(name) and timer_type is None:  # bare decorator
            return self._decorate(name, name.__name__, None, None, None)
        if name is None:
            return lambda fn: self._decorate(fn, fn.__name__, timer_type, cuda_sync, enabled)
        rec = self._get(name, timer_type, cuda_sync, enabled)
        return _TimerHandle(self, rec, name, timer_type, cuda_sync, enabled)

    def _get(self, name, timer_type, cuda_sync, enabled) -> TimerRecord:
        if isinstance(timer_type, str):
            timer_type = TimerType(timer_type)
        if name not in self._timers:
            self._timers[name] = TimerRecord(
                name=name,
                timer_type=timer_type or self._default_type,
                cuda_sync=self._default_sync if cuda_sync is None else cuda_sync,
                enabled=self._enabled if enabled is None else enabled,
            )
        rec = self._timers[name]
        rec.enabled = self._enabled if enabled is None else enabled
        return rec

    def _decorate(self, fn: Callable, name, timer_type, cuda_sync, enabled):
        @wraps(fn)
        def wrapper(*a, **k):
            with self._get(name, timer_type, cuda_sync, enabled):
                return fn(*a, **k)

        return wrapper

    def __getitem__(self, name: str) -> TimerRecord:
        return self._timers[name]

    def __contains__(self, name: str) -> bool:
        return name in self._timers

    def items(self):
        return self._timers.items()

    def reset(self, name: Optional[str] = None):
        if name is None:
            for t in self._timers.values():
                t.reset()
        elif name in self._timers:
            self._timers[name].reset()

    def elapsed(self, name: str) -> float:
        return self._timers[name].elapsed

    def get_all_elapsed(self) -> Dict[str, float]:
        return {n: t.elapsed for n, t in self._timers.items() if t.enabled}

    def log_all(self, logger=None, level=None, rank: Optional[int] = 0):
        import logging

        from nanotron_b200.logging.base import get_logger, log_rank

        logger = logger or get_logger(__name__)
        for n, t in self._timers.items():
            if t.enabled and t.call_count:
                log_rank(f"timer {n}: total {t.total_time*1e3:.2f} ms, avg {t.average_time*1e3:.2f} ms over {t.call_count} calls", logger=logger, level=level or logging.INFO, rank=rank)


class _TimerHandle:
    """Returned by ``timers("x")``: context manager, decorator, and ``start``/``end`` proxy."""

    def __init__(self, owner: Timers, rec: TimerRecord, name, timer_type, cuda_sync, enabled):
        self._owner, self._rec, self._args = owner, rec, (name, timer_type, cuda_sync, enabled)

    def __enter__(self):
        return self._rec.start()

    def __exit__(self, *exc):
        self._rec.end()

    def __call__(self, fn):
        return self._owner._decorate(fn, *self._args)

    def __getattr__(self, item):
        return getattr(self._rec, item)


nanotron_timer = Timers()
