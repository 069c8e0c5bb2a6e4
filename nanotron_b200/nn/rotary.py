"""Rotary position embeddings (parity: reference src/nanotron/nn/rotary.py:11-221).

The cos/sin tables are kept in fp32, indexed by position ids inside the kernel, and applied in place to the q and k
views of the fused qkv projection output, so RoPE costs one read-modify-write of q and k and no extra tensor.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from nanotron_b200 import ops
from nanotron_b200.ops import reference as ref


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, max_seq_len: int, base: float = 10000.0, interleaved: bool = False, seq_len_scaling_factor: Optional[float] = None, fused: bool = True,
                 rope_scaling: Optional[dict] = None):
        super().__init__()
        self.rope_scaling = dict(rope_scaling) if rope_scaling else None
        ref.rope_inverse_frequencies(dim, base, self.rope_scaling)  # an unsupported rule fails here, when the model is built
        self.dim = dim
        self.max_seq_len = max_seq_len
        self.base = base
        self.interleaved = interleaved
        self.seq_len_scaling_factor = seq_len_scaling_factor
        self.fused = fused
        self.register_buffer("cos_table", torch.empty(0), persistent=False)
        self.register_buffer("sin_table", torch.empty(0), persistent=False)

    def _ensure_tables(self, needed_len: int, device):
        if self.cos_table.numel() == 0 or self.cos_table.shape[0] < needed_len or self.cos_table.device != device:
            n = max(needed_len, self.max_seq_len)
            pos = torch.arange(n, device=device)
            cos, sin = ref.rope_cos_sin(pos, self.dim, self.base, self.seq_len_scaling_factor, scaling=self.rope_scaling)
            self.cos_table, self.sin_table = cos.contiguous(), sin.contiguous()

    @property
    def inv_freq(self) -> torch.Tensor:
        return ref.rope_inverse_frequencies(self.dim, self.base, self.rope_scaling)

    def get_cos_sin(self, positions: torch.Tensor, max_position: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos/sin rows [T, dim/2] for flat ``positions`` [T]."""
        self._ensure_tables(max_position if max_position is not None else self.max_seq_len, positions.device)
        idx = positions.reshape(-1).long()
        return self.cos_table.index_select(0, idx), self.sin_table.index_select(0, idx)

    def forward(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor, inplace: bool = False, max_position: Optional[int] = None):
        """q: [T, Hq, D], k: [T, Hkv, D] (views are fine); positions: [T]."""
        self._ensure_tables(max_position if max_position is not None else self.max_seq_len, positions.device)
        pos = positions.reshape(-1)
        q = ops.apply_rotary(q, self.cos_table, self.sin_table, self.interleaved, inplace, positions=pos)
        if k is not None:
            k = ops.apply_rotary(k, self.cos_table, self.sin_table, self.interleaved, inplace, positions=pos)
        return q, k


class FlashRotaryEmbedding(RotaryEmbedding):
    """Same maths; keeps the reference name and its ``seq_len_interpolation_factor`` argument."""

    def __init__(self, dim: int, base: float = 10000.0, interleaved: bool = False, seq_len_interpolation_factor: Optional[float] = None, max_seq_len: int = 4096,
                 rope_scaling: Optional[dict] = None, **_):
        super().__init__(dim=dim, max_seq_len=max_seq_len, base=base, interleaved=interleaved, seq_len_scaling_factor=seq_len_interpolation_factor, rope_scaling=rope_scaling)
