"""Per-module key/value stores for incremental decoding (parity: reference src/nanotron/generation/generate_store.py).

``attach_store(model, store)`` makes every :class:`AttachableStore` sub-module see its own dict inside ``store``
(keyed by module id and pipeline micro-batch); outside the context the modules behave as in training.
"""
from __future__ import annotations

import collections
import contextlib
from typing import Dict, Optional

from torch import nn


class Store(collections.defaultdict):
    """``store[key]`` creates an empty dict on first access."""

    def __init__(self):
        super().__init__(dict)

    def flush(self):
        self.clear()


class AttachableStore:
    def _attach_store(self, store: Store):
        assert not hasattr(self, "_store") or self._store is None, "You can't assign a store when there's already one attached"
        self._store = store

    def _detach_store(self):
        self._store = None

    def get_local_store(self) -> Optional[Dict]:
        store = getattr(self, "_store", None)
        if store is None:
            return None
        return store[id(self)]


def attachable(cls):
    """Class factory: ``cls`` with the AttachableStore mixin (cached per class)."""
    if issubclass(cls, AttachableStore):
        return cls
    name = f"Attachable{cls.__name__}"
    cache = attachable.__dict__.setdefault("_cache", {})
    if cls not in cache:
        cache[cls] = type(name, (cls, AttachableStore), {})
    return cache[cls]


@contextlib.contextmanager
def attach_store(model: nn.Module, store: Store):
    mods = [m for m in model.modules() if isinstance(m, AttachableStore)]
    for m in mods:
        m._attach_store(store)
    try:
        yield
    finally:
        for m in mods:
            m._detach_store()
