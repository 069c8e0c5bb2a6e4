"""Attention backends registry (parity: reference src/nanotron/nn/attention.py:42-238).

All backends take packed tensors q [T, Hq, D], k/v [T, Hkv, D] plus ``cu_seqlens`` and return [T, Hq, D].
``flash_attention_2`` is the in-tree flash attention kernel on CUDA.  ``sdpa`` and ``flex_attention`` are the
PyTorch masked-softmax formulation (document / sliding-window / causal masks).  The ring variants dispatch to
``nanotron_b200.parallel.context_parallel``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from nanotron_b200 import ops
from nanotron_b200.ops import reference as ref


def get_attention_mask(position_ids: torch.Tensor, seq_length: int):
    """Document boundaries from position ids: a 0 starts a new document.  Returns (mask or None, cu_seqlens int32).
    position_ids: [b, s].  Padding positions must be -1."""
    flat = position_ids.reshape(-1)
    starts = torch.nonzero(flat == 0, as_tuple=False).flatten()
    total = torch.tensor([flat.numel()], device=flat.device, dtype=starts.dtype)
    cu = torch.cat([starts, total]).to(torch.int32)
    if cu[0] != 0:
        cu = torch.cat([torch.zeros(1, dtype=torch.int32, device=cu.device), cu])
    return None, cu


def regular_cu_seqlens(batch: int, seq: int, device) -> torch.Tensor:
    return torch.arange(0, (batch + 1) * seq, seq, dtype=torch.int32, device=device)


def flash_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, **_):
    return ops.flash_attn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=causal, softmax_scale=softmax_scale, window=sliding_window)


def sdpa_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, **_):
    return ref.attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=causal, softmax_scale=softmax_scale, window=sliding_window)


def flex_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, flex_attention_mask: Optional[str] = None, **_):
    """Mask kinds "sliding_window", "document", "sliding_window_document" map onto (cu_seqlens, window)."""
    if flex_attention_mask == "sliding_window":
        total_q = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
        total_k = torch.tensor([0, k.shape[0]], dtype=torch.int32, device=q.device)
        return ref.attention_varlen(q, k, v, total_q, total_k, causal=causal, softmax_scale=softmax_scale, window=sliding_window)
    window = sliding_window if flex_attention_mask in ("sliding_window_document",) or flex_attention_mask is None else None
    return ref.attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=causal, softmax_scale=softmax_scale, window=window)


def _ring(kind: str) -> Callable:
    def fn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, cp_pg=None, **kw):
        from nanotron_b200.parallel.context_parallel.ring_attention import ring_attention

        return ring_attention(q, k, v, cp_pg=cp_pg, causal=causal, softmax_scale=softmax_scale, variant=kind, **kw)

    return fn


ALL_ATTENTION_FUNCTIONS: Dict[str, Callable] = {
    "flash_attention_2": flash_attention_forward,
    "flex_attention": flex_attention_forward,
    "sdpa": sdpa_attention_forward,
    "ring_flash_triton": _ring("ring"),
    "ring": _ring("ring"),
    "llama3_ring_attention": _ring("allgather"),
    "ring_fused": _ring("fused"),
}
AttentionImplementation = str
