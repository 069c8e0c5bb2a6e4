"""Quantised copies of weights that live as long as the weights do not change
(scope parity: reference src/nanotron/fp8/parameter.py, whose ``FP8Parameter`` keeps an fp8 payload next to the parameter).

A weight is read by the forward and by the dgrad of EVERY micro-batch but only changes at the optimizer step, so its
128 x 128-block e4m3 copy (and the transposed copy the K-major dgrad kernel wants) is computed once per optimizer step and
looked up afterwards.  An entry is valid while the cache's *generation* and the tensor's autograd version are the ones it was
made under.  The trainer starts a new generation after every optimizer step and after loading weights: the fused optimizer
kernels write parameters through raw pointers, which autograd's version counter does not see; in-place PyTorch updates are
caught by the version counter as well.
"""
from __future__ import annotations

import weakref
from typing import Dict, Tuple

import torch

from nanotron_b200.fp8.quantize import FP8BlockTensor, quantize_128x128


class QuantizedWeightCache:
    def __init__(self):
        self.generation = 0
        self.enabled = True
        self.hits = 0
        self.misses = 0
        self._entries: Dict[Tuple, Tuple] = {}  # key -> (generation, version, copy, weak reference to the source tensor)

    def invalidate(self) -> None:
        """The weights changed (optimizer step, checkpoint load): forget every quantised copy."""
        self.generation += 1
        self._entries.clear()

    def get(self, weight: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn, transposed: bool = False) -> FP8BlockTensor:
        """128 x 128-block copy of ``weight`` ([N, K]); ``transposed``: of ``weight.t()`` ([K, N], payload and scales transposed)."""
        if not self.enabled:
            q = quantize_128x128(weight, dtype)
            return _transpose(q) if transposed else q
        key = (weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()), weight.dtype, dtype, transposed)
        hit = self._entries.get(key)
        if hit is not None and hit[0] == self.generation and hit[1] == weight._version:
            owner = hit[3]()  # the tensor the copy was made from must still be alive at this address: a freed weight's
            if owner is not None and owner.data_ptr() == weight.data_ptr():  # memory may have been handed to another tensor
                self.hits += 1
                return hit[2]
        self.misses += 1
        if transposed:
            q = _transpose(self.get(weight, dtype, transposed=False))
        else:
            with torch.no_grad():
                q = quantize_128x128(weight.detach(), dtype)
        self._entries[key] = (self.generation, weight._version, q, weakref.ref(weight))
        return q


def _transpose(q: FP8BlockTensor) -> FP8BlockTensor:
    return FP8BlockTensor(q.data.t().contiguous(), q.scale.t().contiguous(), q.block)


weight_cache = QuantizedWeightCache()


class FP8Parameter(torch.nn.Parameter):
    """A parameter that hands out its own block-quantised copy (``.fp8`` / ``.fp8_t``) through the shared cache."""

    @property
    def fp8(self) -> FP8BlockTensor:
        return weight_cache.get(self)

    @property
    def fp8_t(self) -> FP8BlockTensor:
        return weight_cache.get(self, transposed=True)
