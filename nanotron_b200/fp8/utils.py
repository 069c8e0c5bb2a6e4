"""Small helpers around fp8 tensors (scope parity: reference src/nanotron/fp8/utils.py)."""
from __future__ import annotations

from typing import Dict

import torch

from nanotron_b200.fp8.constants import FP8_MAX
from nanotron_b200.fp8.dtypes import DTypes


def is_overflow_underflow_nan(tensor: torch.Tensor) -> bool:
    """True when a tensor carries inf or nan (what an fp8 cast without a fitting scale produces)."""
    return bool(torch.isinf(tensor).any() or torch.isnan(tensor).any())


def quantization_error(reference: torch.Tensor, quantised: torch.Tensor) -> Dict[str, float]:
    """How far a dequantised tensor is from its source: worst relative error against the largest magnitude, and signal-to-noise in dB."""
    ref, q = reference.float(), quantised.float()
    err = (ref - q).abs()
    noise = err.pow(2).mean().clamp(min=1e-30)
    return {"max_rel": float(err.max() / ref.abs().max().clamp(min=1e-30)), "snr_db": float(10 * torch.log10(ref.pow(2).mean().clamp(min=1e-30) / noise))}


def representable_range(dtype: DTypes) -> float:
    return FP8_MAX[dtype]
