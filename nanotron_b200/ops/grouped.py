"""Grouped expert MLP on CUDA: rows of ``x_sorted`` are grouped by local expert, ``counts[e]`` rows each.

y = (swiglu(x_e @ W_gate_up[e])) @ W_down[e] for every expert, with device-side group offsets (no host
synchronisation on the token counts, unlike reference src/nanotron/nn/moe.py:93 which moves them to the CPU).
The two grouped products currently go through the library grouped GEMM (``torch._grouped_mm``); the SwiGLU between them
is the in-tree kernel.  A tcgen05 grouped GEMM with a masked epilogue is the planned replacement.
"""
from __future__ import annotations

import torch

from nanotron_b200 import ops


def grouped_mlp(x_sorted: torch.Tensor, counts: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    offs = torch.cumsum(counts, dim=0).to(torch.int32)
    if x_sorted.shape[0] == 0:
        return x_sorted.new_zeros((0, w_down.shape[-1]))
    if hasattr(torch, "_grouped_mm") and x_sorted.dtype == torch.bfloat16 and x_sorted.shape[1] % 8 == 0:
        h = torch._grouped_mm(x_sorted, w_gate_up, offs=offs)
        a = ops.swiglu(h)
        return torch._grouped_mm(a, w_down, offs=offs)
    from nanotron_b200.nn.moe import grouped_mlp_reference

    return grouped_mlp_reference(x_sorted, counts, w_gate_up, w_down)
