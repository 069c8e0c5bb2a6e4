"""The number formats of the fp8 path (scope parity: reference src/nanotron/fp8/dtypes.py)."""
from enum import Enum

import torch


class DTypes(Enum):
    FP8E4M3 = "fp8e4m3"   # forward tensors: 4 exponent bits, max 448
    FP8E5M2 = "fp8e5m2"   # gradients: 5 exponent bits, max 57344
    KFLOAT16 = "kfloat16"
    KBFLOAT16 = "kbfloat16"
    KFLOAT32 = "kfloat32"

    @property
    def torch_dtype(self) -> torch.dtype:
        return _TORCH[self]

    @classmethod
    def of(cls, dtype: torch.dtype) -> "DTypes":
        return next(k for k, v in _TORCH.items() if v == dtype)


_TORCH = {
    DTypes.FP8E4M3: torch.float8_e4m3fn,
    DTypes.FP8E5M2: torch.float8_e5m2,
    DTypes.KFLOAT16: torch.float16,
    DTypes.KBFLOAT16: torch.bfloat16,
    DTypes.KFLOAT32: torch.float32,
}
