"""Per-tensor scaled fp8 tensors with power-of-two scales (scope parity: reference src/nanotron/fp8/tensor.py:77-105, which
casts through TransformerEngine; here the cast is PyTorch's own fp8 dtypes, so it also runs on CPU).

``scale = 2 ** (floor(log2(max / amax)) - margin)``: a power of two changes only the exponent of every element, so scaling
and unscaling are exact and the rounding error is the format's alone.  The block-scaled tensors of ``quantize.py`` are what
the training path uses; these are for tools, checkpoints and comparisons that want one scale per tensor.
"""
from __future__ import annotations

import math
from typing import Union

import torch

from nanotron_b200.fp8.constants import DEFAULT_MARGIN, FP8_MAX
from nanotron_b200.fp8.dtypes import DTypes
from nanotron_b200.fp8.meta import FP8Meta


def compute_scale(amax: torch.Tensor, dtype: DTypes, margin: int = DEFAULT_MARGIN) -> torch.Tensor:
    """Largest power of two that keeps ``amax * scale`` inside the format (1 for an all-zero or non-finite tensor)."""
    a = float(amax)
    if not math.isfinite(a) or a <= 0.0:
        return torch.tensor(1.0, dtype=torch.float32, device=amax.device)
    exponent = math.floor(math.log2(FP8_MAX[dtype] / a)) - margin
    return torch.tensor(2.0**exponent, dtype=torch.float32, device=amax.device)


class FP8Tensor:
    """fp8 payload + :class:`FP8Meta`.  ``FP8Tensor(x, DTypes.FP8E4M3)`` quantises; ``.to_float()`` gives the values back."""

    def __init__(self, tensor: torch.Tensor, dtype: Union[DTypes, torch.dtype] = DTypes.FP8E4M3, margin: int = DEFAULT_MARGIN, interval: int = 1):
        dtype = dtype if isinstance(dtype, DTypes) else DTypes.of(dtype)
        assert dtype in FP8_MAX, f"{dtype} is not an fp8 format"
        assert tensor.dtype not in (torch.int8, torch.uint8), "expected a floating-point tensor"
        amax = tensor.detach().abs().amax().float() if tensor.numel() else torch.zeros((), device=tensor.device)
        self.fp8_meta = FP8Meta(amax=amax, scale=compute_scale(amax, dtype, margin), dtype=dtype, interval=interval)
        self.data = self._cast(tensor)

    def _cast(self, tensor: torch.Tensor) -> torch.Tensor:
        m = self.fp8_meta
        return (tensor.detach().float() * m.scale).clamp(-m.fp8_max, m.fp8_max).to(m.dtype.torch_dtype)

    @property
    def shape(self):
        return self.data.shape

    def to_float(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return (self.data.float() * self.fp8_meta.inverse_scale).to(dtype)

    def set_data(self, tensor: torch.Tensor) -> None:
        """New contents; the scale is kept unless the new maximum no longer fits it (or wastes range)."""
        amax = tensor.detach().abs().amax().float()
        if self.fp8_meta.needs_rescale(amax):
            self.fp8_meta.scale = compute_scale(amax, self.fp8_meta.dtype)
        self.fp8_meta.amax = amax
        self.data = self._cast(tensor)


def convert_tensor_from_fp8(data: torch.Tensor, meta: FP8Meta, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return (data.float() * meta.inverse_scale).to(dtype)
