"""Named random-number-generator states: capture, install, branch into for the length of a block, and copy from one rank to a
group (API parity: reference src/nanotron/random.py:13-148).

A ``RandomState`` is a snapshot of the four generators a training process draws from (Python, NumPy, torch CPU, torch CUDA).
The snapshot knows how to take itself (``RandomState.capture``) and how to put itself back (``install``); the module-level
functions of the reference API are thin names for those.  The CUDA part is ``None`` on machines without a GPU, which is what
lets the same code run under gloo on CPU.
"""
from __future__ import annotations

import contextlib
import random
from dataclasses import dataclass, fields
from typing import Dict, Iterator, MutableMapping, Optional, Tuple

import numpy as np
import torch

import nanotron_b200.distributed as dist


def _same(a, b) -> bool:
    """Equality over the kinds of values generator states are made of."""
    if a is None or b is None:
        return a is None and b is None
    if torch.is_tensor(a):
        return torch.is_tensor(b) and torch.equal(a, b)
    if isinstance(a, np.ndarray):
        return isinstance(b, np.ndarray) and np.array_equal(a, b)
    if isinstance(a, (tuple, list)):
        return isinstance(b, (tuple, list)) and len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    return a == b


@dataclass
class RandomState:
    random: Tuple
    numpy: Tuple
    torch_cpu: torch.Tensor
    torch_cuda: Optional[torch.Tensor]

    @classmethod
    def capture(cls) -> "RandomState":
        cuda = torch.cuda.get_rng_state("cuda") if torch.cuda.is_available() else None
        return cls(random=random.getstate(), numpy=np.random.get_state(), torch_cpu=torch.random.get_rng_state(), torch_cuda=cuda)

    def install(self) -> None:
        random.setstate(self.random)
        np.random.set_state(self.numpy)
        torch.set_rng_state(self.torch_cpu)
        if self.torch_cuda is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(self.torch_cuda, "cuda")

    def __eq__(self, other):
        return isinstance(other, RandomState) and all(_same(getattr(self, f.name), getattr(other, f.name)) for f in fields(self))


class RandomStates(MutableMapping[str, RandomState]):
    """A fixed set of named states: values can be replaced, names can neither be added nor removed after construction."""

    def __init__(self, dict: Dict[str, RandomState]):
        for name, state in dict.items():
            self.check_type(name, state)
        self._dict = dict

    @staticmethod
    def check_type(key, value):
        if not isinstance(key, str):
            raise ValueError(f"Expected key to be of type str. Got {type(key)}")
        if not isinstance(value, RandomState):
            raise ValueError(f"Expected value to be of type `RandomState`. Got {type(value)}")

    def __getitem__(self, name: str) -> RandomState:
        return self._dict[name]

    def __setitem__(self, name: str, state: RandomState):
        if name not in self._dict:
            raise ValueError("Can't add a new random states after initialisation")
        self.check_type(name, state)
        self._dict[name] = state

    def __delitem__(self, name: str):
        raise ValueError("Can't delete a random states key")

    def __iter__(self) -> Iterator[str]:
        return iter(self._dict)

    def __len__(self) -> int:
        return len(self._dict)

    def __eq__(self, other):
        return isinstance(other, RandomStates) and self._dict == other._dict


def set_random_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def set_random_state(random_state: RandomState):
    random_state.install()


def get_current_random_state() -> RandomState:
    return RandomState.capture()


@contextlib.contextmanager
def branch_random_state(random_states: RandomStates, key: str, enabled: bool):
    """The body draws from ``random_states[key]``; what is left of that stream afterwards is stored back under the same name and
    the generators return to where they were before the block."""
    if not enabled:
        yield
        return
    ambient = RandomState.capture()
    random_states[key].install()
    try:
        yield
    finally:
        random_states[key] = RandomState.capture()
        ambient.install()


def get_synced_random_state(random_state: RandomState, pg: dist.ProcessGroup) -> RandomState:
    """Every rank of ``pg`` leaves with the state of the group's first rank."""
    first = dist.get_global_rank(pg, 0)
    box = [random_state if dist.get_rank(pg) == 0 else None]
    device = torch.device("cuda") if dist.get_backend() == "nccl" else torch.device("cpu")
    dist.broadcast_object_list(box, src=first, group=pg, device=device)
    synced: RandomState = box[0]
    if synced.torch_cuda is not None:
        synced.torch_cuda = synced.torch_cuda.cpu()  # generator states live on the host wherever they were pickled
    return synced
