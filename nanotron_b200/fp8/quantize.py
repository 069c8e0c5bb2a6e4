"""Block-scaled fp8 tensors (scope parity: reference src/nanotron/fp8/{tensor,meta,constants}.py, which only has per-tensor
scaling through TransformerEngine and is not wired into any model).

Scaling granularity: activations and gradients 1 x 128 (one scale per row per 128 columns), weights 128 x 128.
Forward tensors use e4m3 (max 448), gradients e5m2 (max 57344).  Scales are fp32 ``amax / fmax`` (dequantised value =
payload * scale).  On CUDA the quantisation is one in-tree kernel pass; on CPU it is the PyTorch restatement below, which
is also the oracle for the kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
BLOCK = 128


def _fmax(dtype: torch.dtype) -> float:
    return E4M3_MAX if dtype == torch.float8_e4m3fn else E5M2_MAX


@dataclass
class FP8BlockTensor:
    data: torch.Tensor   # fp8 payload, same shape as the source
    scale: torch.Tensor  # fp32 [rows, cols/128] (1x128) or [rows/128, cols/128] (128x128)
    block: Tuple[int, int]

    @property
    def shape(self):
        return self.data.shape


def _pad_to(x: torch.Tensor, m0: int, m1: int) -> torch.Tensor:
    r, c = x.shape
    pr, pc = (-r) % m0, (-c) % m1
    if pr or pc:
        x = torch.nn.functional.pad(x, (0, pc, 0, pr))
    return x


def quantize_1x128_reference(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> FP8BlockTensor:
    rows, cols = x.shape
    xp = _pad_to(x.float(), 1, BLOCK)
    blocks = xp.view(rows, -1, BLOCK)
    amax = blocks.abs().amax(dim=-1).clamp(min=1e-12)
    scale = amax / _fmax(dtype)
    q = (blocks / scale.unsqueeze(-1)).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype)
    return FP8BlockTensor(q.view(rows, -1)[:, :cols].contiguous(), scale.contiguous(), (1, BLOCK))


def quantize_128x128_reference(w: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> FP8BlockTensor:
    rows, cols = w.shape
    wp = _pad_to(w.float(), BLOCK, BLOCK)
    R, C = wp.shape
    blocks = wp.view(R // BLOCK, BLOCK, C // BLOCK, BLOCK).permute(0, 2, 1, 3)
    amax = blocks.abs().amax(dim=(-1, -2)).clamp(min=1e-12)
    scale = amax / _fmax(dtype)
    q = (blocks / scale[..., None, None]).clamp(-_fmax(dtype), _fmax(dtype)).to(dtype)
    q = q.permute(0, 2, 1, 3).reshape(R, C)[:rows, :cols].contiguous()
    return FP8BlockTensor(q, scale.contiguous(), (BLOCK, BLOCK))


def quantize_1x128(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> FP8BlockTensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % BLOCK == 0 and x.is_contiguous():
        from nanotron_b200 import ops
        from nanotron_b200.ops import native

        if ops.get_mode() != "torch" and native.has_fp8_quantize():
            return native.fp8_quantize_1x128(x, dtype)
    return quantize_1x128_reference(x, dtype)


def quantize_128x128(w: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> FP8BlockTensor:
    return quantize_128x128_reference(w, dtype)  # weights are quantised once per step: not a hot path


def dequantize(t: FP8BlockTensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    rows, cols = t.data.shape
    x = t.data.float()
    br, bc = t.block
    s = t.scale
    s = s.repeat_interleave(bc, dim=1)[:, :cols]
    if br > 1:
        s = s.repeat_interleave(br, dim=0)[:rows]
    return (x * s).to(dtype)
