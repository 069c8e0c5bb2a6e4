"""Named RNG states that can be branched into and synchronised over a group (parity: reference src/nanotron/random.py)."""
from __future__ import annotations

import contextlib
import random
from dataclasses import dataclass
from typing import MutableMapping, Optional, Tuple

import numpy as np
import torch

import nanotron_b200.distributed as dist


@dataclass
class RandomState:
    random: Tuple
    numpy: Tuple
    torch_cpu: torch.Tensor
    torch_cuda: Optional[torch.Tensor]

    def __eq__(self, other):
        return (
            isinstance(other, RandomState)
            and self.random == other.random
            and all(np.array_equal(a, b) if isinstance(a, np.ndarray) else a == b for a, b in zip(self.numpy, other.numpy))
            and torch.equal(self.torch_cpu, other.torch_cpu)
            and ((self.torch_cuda is None and other.torch_cuda is None) or (self.torch_cuda is not None and other.torch_cuda is not None and torch.equal(self.torch_cuda, other.torch_cuda)))
        )


class RandomStates(MutableMapping[str, RandomState]):
    def __init__(self, dict: dict):
        for k, v in dict.items():
            self.check_type(k, v)
        self._dict = dict

    @staticmethod
    def check_type(key, value):
        if not isinstance(key, str):
            raise ValueError(f"Expected key to be of type str. Got {type(key)}")
        if not isinstance(value, RandomState):
            raise ValueError(f"Expected value to be of type `RandomState`. Got {type(value)}")

    def __getitem__(self, item):
        return self._dict[item]

    def __iter__(self):
        return iter(self._dict)

    def __len__(self):
        return len(self._dict)

    def __delitem__(self, key):
        raise ValueError("Can't delete a random states key")

    def __setitem__(self, key, value):
        if key not in self._dict:
            raise ValueError("Can't add a new random states after initialisation")
        self.check_type(key, value)
        self._dict[key] = value

    def __eq__(self, other):
        return isinstance(other, RandomStates) and self._dict == other._dict


def set_random_seed(seed: int):
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def set_random_state(random_state: RandomState):
    random.setstate(random_state.random)
    np.random.set_state(random_state.numpy)
    torch.set_rng_state(random_state.torch_cpu)
    if torch.cuda.is_available() and random_state.torch_cuda is not None:
        torch.cuda.set_rng_state(random_state.torch_cuda, "cuda")


def get_current_random_state() -> RandomState:
    return RandomState(
        random=random.getstate(),
        numpy=np.random.get_state(),
        torch_cpu=torch.random.get_rng_state(),
        torch_cuda=torch.cuda.get_rng_state("cuda") if torch.cuda.is_available() else None,
    )


@contextlib.contextmanager
def branch_random_state(random_states: RandomStates, key: str, enabled: bool):
    """Run the body under ``random_states[key]`` and store the advanced state back; the ambient state is restored."""
    if not enabled:
        yield
        return
    old = get_current_random_state()
    set_random_state(random_states[key])
    try:
        yield
    finally:
        random_states[key] = get_current_random_state()
        set_random_state(old)


def get_synced_random_state(random_state: RandomState, pg: dist.ProcessGroup) -> RandomState:
    """Every rank of ``pg`` receives rank 0's state."""
    reference_rank = 0
    if dist.get_rank(pg) == reference_rank:
        obj = [random_state]
    else:
        obj = [None]
    dist.broadcast_object_list(obj, src=dist.get_global_rank(pg, reference_rank), group=pg, device=torch.device("cuda") if dist.get_backend() == "nccl" else torch.device("cpu"))
    new = obj[0]
    if new.torch_cuda is not None:
        new.torch_cuda = new.torch_cuda.cpu()
    return new
