"""Scaling metadata of a per-tensor fp8 tensor (scope parity: reference src/nanotron/fp8/meta.py)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from nanotron_b200.fp8.constants import DEFAULT_INTERVAL, FP8_MAX
from nanotron_b200.fp8.dtypes import DTypes


@dataclass
class FP8Meta:
    amax: torch.Tensor   # fp32 scalar: largest magnitude the scale was derived from
    scale: torch.Tensor  # fp32 scalar, a power of two: payload = value * scale
    dtype: DTypes
    interval: int = DEFAULT_INTERVAL  # steps between refreshes of the scale

    @property
    def fp8_max(self) -> float:
        return FP8_MAX[self.dtype]

    @property
    def inverse_scale(self) -> torch.Tensor:
        return 1.0 / self.scale

    def needs_rescale(self, new_amax: torch.Tensor) -> bool:
        """True when a tensor with maximum ``new_amax`` would overflow the format under the current scale, or waste more than one
        bit of its range."""
        scaled = float(new_amax) * float(self.scale)
        return scaled > self.fp8_max or scaled < self.fp8_max / 4
