"""Attention backends registry (parity: reference src/nanotron/nn/attention.py:42-238).

All backends take packed tensors q [T, Hq, D], k/v [T, Hkv, D] plus ``cu_seqlens`` and return [T, Hq, D].
``flash_attention_2``, ``sdpa`` and ``flex_attention`` all end in ``ops.flash_attn_varlen``: the in-tree flash attention kernel on
CUDA (document / sliding-window / causal masks are its native inputs), the fp32 masked-softmax oracle on CPU.  The ring variants dispatch to
``nanotron_b200.parallel.context_parallel``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from nanotron_b200 import ops


def get_attention_mask(position_ids: torch.Tensor, seq_length: int):
    """Document boundaries from position ids: a 0 starts a new document, and so does the first token of every batch row (a row
    that begins in the middle of a document must not see the end of the previous row; the reference cuts at zeros only,
    src/nanotron/nn/attention.py:227-238).  Returns (mask or None, cu_seqlens int32).  position_ids: [b, s]."""
    is_start = position_ids == 0
    is_start[:, 0] = True
    starts = torch.nonzero(is_start.reshape(-1), as_tuple=False).flatten()
    total = torch.tensor([position_ids.numel()], device=starts.device, dtype=starts.dtype)
    return None, torch.cat([starts, total]).to(torch.int32)


def regular_cu_seqlens(batch: int, seq: int, device) -> torch.Tensor:
    return torch.arange(0, (batch + 1) * seq, seq, dtype=torch.int32, device=device)


def flash_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, **_):
    return ops.flash_attn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=causal, softmax_scale=softmax_scale, window=sliding_window)


def sdpa_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, **_):
    """The "sdpa" backend name of the reference (src/nanotron/nn/attention.py:200-209).  Same computation as ``flash_attention_2``:
    CUDA tensors run the in-tree kernel (or, outside its contract, the library kernel with an explicit mask), CPU tensors the
    fp32 masked-softmax oracle."""
    return ops.flash_attn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=causal, softmax_scale=softmax_scale, window=sliding_window)


def flex_attention_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=True, softmax_scale=None, sliding_window=None, flex_attention_mask: Optional[str] = None, softcap: Optional[float] = None, **_):
    """Mask-programmable attention (reference src/nanotron/nn/attention.py:120-129 + nn/flex_attention.py).  The mask kinds the
    reference builds block masks for -- "causal", "sliding_window", "document", "sliding_window_document" -- are all of the form
    (document boundaries, causal, window), which is what the in-tree kernel takes directly: ``nn.flex_attention.BlockMask``
    carries that description instead of a dense block table.  Score soft-capping has no kernel and runs the fp32 formulation."""
    from nanotron_b200.nn.flex_attention import block_mask_for

    bm = block_mask_for(flex_attention_mask, cu_seqlens_q, cu_seqlens_k, total_q=q.shape[0], total_k=k.shape[0], max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, causal=causal, sliding_window=sliding_window)
    if softcap is not None:
        from nanotron_b200.nn.flex_attention import softcapped_attention

        return softcapped_attention(q, k, v, bm, softcap=softcap, softmax_scale=softmax_scale)
    return ops.flash_attn_varlen(q, k, v, bm.cu_seqlens_q, bm.cu_seqlens_k, bm.max_seqlen_q, bm.max_seqlen_k, causal=bm.causal, softmax_scale=softmax_scale, window=bm.window)


def _packed_index(mask: torch.Tensor):
    """(flat indices of the True positions, cu_seqlens int32 [b + 1]) of a [b, n] mask; cached on the mask tensor because every
    layer of a decoding step asks for the same one (building it reads the mask back on the host once)."""
    cached = getattr(mask, "_ntb_packed_index", None)
    if cached is not None:
        return cached
    m = mask.bool()
    idx = torch.nonzero(m.reshape(-1), as_tuple=False).flatten()
    cu = torch.cat([torch.zeros(1, dtype=torch.int32, device=m.device), m.sum(-1).cumsum(0).to(torch.int32)])
    try:
        mask._ntb_packed_index = (idx, cu)
    except AttributeError:
        pass
    return idx, cu


def cached_attention(q: torch.Tensor, k_all: torch.Tensor, v_all: torch.Tensor, q_mask: torch.Tensor, kv_mask: torch.Tensor, softmax_scale: Optional[float] = None, sliding_window: Optional[int] = None) -> torch.Tensor:
    """Attention of the new positions against the key/value cache (decoding; reference: ``flash_attn_with_kvcache`` call sites,
    src/nanotron/models/llama.py:645-658, starcoder2.py:832,1077).

    q: [b, q_len, Hq, D] (the positions being decoded now); k_all, v_all: [b, kv_len, Hkv, D] (cache including the new positions);
    q_mask [b, q_len], kv_mask [b, kv_len]: which entries are real tokens (left padding on the first call).  The real queries of
    a row are the LAST real keys of that row, which is what the bottom-right aligned causal mask of the variable-length kernel
    expresses, so padded batches are packed and handed to ``ops.flash_attn_varlen`` (in-tree kernel on CUDA).  Returns
    [b, q_len, Hq, D] with zeros at padded query positions."""
    b, q_len, Hq, D = q.shape
    kv_len = k_all.shape[1]
    qi, cu_q = _packed_index(q_mask)
    ki, cu_k = _packed_index(kv_mask)
    qp = q.reshape(b * q_len, Hq, D).index_select(0, qi)
    kp = k_all.reshape(b * kv_len, k_all.shape[2], D).index_select(0, ki)
    vp = v_all.reshape(b * kv_len, v_all.shape[2], D).index_select(0, ki)
    op = ops.flash_attn_varlen(qp, kp, vp, cu_q, cu_k, q_len, kv_len, causal=True, softmax_scale=softmax_scale, window=sliding_window)
    out = torch.zeros((b * q_len, Hq, D), dtype=op.dtype, device=q.device)
    out.index_copy_(0, qi, op)
    return out.view(b, q_len, Hq, D)


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
