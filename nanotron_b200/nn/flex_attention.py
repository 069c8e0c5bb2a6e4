"""Mask descriptions for the programmable-mask attention backend (capability parity: reference
src/nanotron/nn/flex_attention.py:12-403, which builds PyTorch FlexAttention block masks from Python predicates).

Every mask the reference can express is a conjunction of three terms: *same document*, *causal*, *within a sliding window*.
The in-tree attention kernels take exactly these as inputs (``cu_seqlens`` for the documents, a causal flag, a window
length) and skip whole 128 x 128 key tiles that the terms rule out, so a mask here is a small value object, ``BlockMask``,
rather than a dense table of blocks.  What the reference caches with ``functools.lru_cache`` (block tables per predicate and
shape) is cached here per (kind, boundaries, shape) as well, because building ``cu_seqlens`` from position ids costs a
device round trip.

``BlockMask.block_table`` materialises the classic block-sparsity summary (0 = skipped, 1 = partially masked, 2 = full tile)
for inspection and for tests; the kernels never read it.
"""
from __future__ import annotations

import dataclasses
import functools
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch

BLOCK = 128
MASK_KINDS = ("causal", "full", "sliding_window", "document", "sliding_window_document")


@dataclasses.dataclass(frozen=True, eq=False)
class BlockMask:
    cu_seqlens_q: torch.Tensor  # int32 [n_docs + 1]
    cu_seqlens_k: torch.Tensor
    max_seqlen_q: int
    max_seqlen_k: int
    causal: bool = True
    window: Optional[int] = None  # a query sees at most this many keys, itself included

    def mask_mod(self) -> Callable[[int, int], bool]:
        """``f(q_idx, kv_idx) -> bool`` over flat token indices, for checking a mask element by element."""
        cq, ck = self.cu_seqlens_q.tolist(), self.cu_seqlens_k.tolist()

        def f(qi: int, ki: int) -> bool:
            d = next((d for d in range(len(cq) - 1) if cq[d] <= qi < cq[d + 1]), None)
            if d is None or not (ck[d] <= ki < ck[d + 1]):
                return False
            lq, lk = cq[d + 1] - cq[d], ck[d + 1] - ck[d]
            i, j = qi - cq[d] + (lk - lq), ki - ck[d]  # bottom-right aligned
            if self.causal and j > i:
                return False
            if self.window and j <= i - self.window:
                return False
            return True

        return f

    def dense(self) -> torch.Tensor:
        """Boolean [total_q, total_k] mask (True = attend); O(T^2) memory, for tests and small inputs only."""
        cq, ck = self.cu_seqlens_q.tolist(), self.cu_seqlens_k.tolist()
        dev = self.cu_seqlens_q.device
        m = torch.zeros(cq[-1], ck[-1], dtype=torch.bool, device=dev)
        for d in range(len(cq) - 1):
            lq, lk = cq[d + 1] - cq[d], ck[d + 1] - ck[d]
            if lq == 0 or lk == 0:
                continue
            i = torch.arange(lq, device=dev).unsqueeze(1) + (lk - lq)
            j = torch.arange(lk, device=dev).unsqueeze(0)
            sub = torch.ones(lq, lk, dtype=torch.bool, device=dev)
            if self.causal:
                sub &= j <= i
            if self.window:
                sub &= j > i - self.window
            m[cq[d] : cq[d + 1], ck[d] : ck[d + 1]] = sub
        return m

    def block_table(self, block: int = BLOCK) -> torch.Tensor:
        """int8 [ceil(Tq / block), ceil(Tk / block)]: 0 = no element attends (tile skipped), 2 = every element attends, 1 = mixed."""
        d = self.dense()
        tq, tk = d.shape
        nq, nk = -(-tq // block), -(-tk // block)
        padded = torch.zeros(nq * block, nk * block, dtype=torch.bool, device=d.device)
        padded[:tq, :tk] = d
        tiles = padded.view(nq, block, nk, block).permute(0, 2, 1, 3).reshape(nq, nk, -1)
        valid = torch.zeros(nq * block, nk * block, dtype=torch.bool, device=d.device)
        valid[:tq, :tk] = True
        valid = valid.view(nq, block, nk, block).permute(0, 2, 1, 3).reshape(nq, nk, -1)
        any_, all_ = tiles.any(-1), (tiles | ~valid).all(-1)
        return (any_.to(torch.int8) + (any_ & all_).to(torch.int8))

    def sparsity(self, block: int = BLOCK) -> float:
        """Fraction of key tiles the kernel skips."""
        t = self.block_table(block)
        return float((t == 0).float().mean())


# ---------------------------------------------------------------------------- document boundaries
def lengths_to_offsets(lengths: Union[Sequence[int], torch.Tensor], device=None) -> torch.Tensor:
    """Document lengths -> cumulative offsets, int32 [n + 1] starting at 0."""
    t = lengths if isinstance(lengths, torch.Tensor) else torch.tensor(list(lengths), dtype=torch.int32, device=device)
    t = t.to(device=device if device is not None else t.device, dtype=torch.int32)
    return torch.cat([torch.zeros(1, dtype=torch.int32, device=t.device), torch.cumsum(t, 0).to(torch.int32)])


def offsets_to_doc_ids(offsets: torch.Tensor) -> torch.Tensor:
    """Offsets [n + 1] -> document id of every token, int32 [offsets[-1]]."""
    counts = (offsets[1:] - offsets[:-1]).long()
    return torch.repeat_interleave(torch.arange(counts.numel(), device=offsets.device, dtype=torch.int32), counts)


def doc_ids_to_offsets(document_ids: torch.Tensor) -> torch.Tensor:
    """Per-token document ids (non-decreasing runs) -> offsets [n + 1]."""
    flat = document_ids.reshape(-1)
    change = torch.nonzero(flat[1:] != flat[:-1], as_tuple=False).flatten() + 1
    return torch.cat([torch.zeros(1, dtype=torch.int64, device=flat.device), change, torch.tensor([flat.numel()], device=flat.device)]).to(torch.int32)


def position_ids_to_offsets(position_ids: torch.Tensor) -> torch.Tensor:
    """Packed position ids ([b, s] or [T]; a 0 starts a document, rows of a batch are separate documents) -> offsets."""
    if position_ids.dim() == 2:
        b, s = position_ids.shape
        flat = position_ids.reshape(-1)
        starts = (flat == 0)
        starts[torch.arange(0, b * s, s, device=flat.device)] = True
    else:
        flat = position_ids
        starts = flat == 0
        starts[0] = True
    idx = torch.nonzero(starts, as_tuple=False).flatten()
    return torch.cat([idx, torch.tensor([flat.numel()], device=flat.device)]).to(torch.int32)


# ---------------------------------------------------------------------------- builders
def _one_document(total: int, device) -> torch.Tensor:
    return torch.tensor([0, total], dtype=torch.int32, device=device)


def create_attention_mask(total_q: int, total_k: Optional[int] = None, *, offsets: Optional[torch.Tensor] = None, document_ids: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None, sliding_window: Optional[int] = None, causal: bool = True, device=None) -> BlockMask:
    """The reference's ``create_attention_mask`` (nn/flex_attention.py:89-135) over this module's mask object: documents from
    ``offsets``, ``document_ids`` or ``position_ids`` (none of them: one document), optional window, causal by default."""
    total_k = total_q if total_k is None else total_k
    if offsets is None and document_ids is not None:
        offsets = doc_ids_to_offsets(document_ids)
    if offsets is None and position_ids is not None:
        offsets = position_ids_to_offsets(position_ids)
    if offsets is None:
        cq, ck = _one_document(total_q, device), _one_document(total_k, device)
        mq, mk = total_q, total_k
    else:
        assert total_q == total_k, "document masks need the same packing for queries and keys"
        cq = ck = offsets.to(torch.int32)
        mq = mk = int((cq[1:] - cq[:-1]).max())
    return BlockMask(cq, ck, mq, mk, causal=causal, window=sliding_window or None)


_CACHE: dict = {}
_CACHE_ORDER: List[Tuple] = []
_CACHE_SIZE = 32


def block_mask_for(kind: Optional[str], cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, total_q: int, total_k: int, max_seqlen_q: int, max_seqlen_k: int, causal: bool = True, sliding_window: Optional[int] = None) -> BlockMask:
    """Mask object for one of the named kinds (``MASK_KINDS``; None means "whatever the inputs say": documents + window).
    "sliding_window" and "causal" ignore document boundaries, "document" ignores the window.  Results are cached on the
    identity of the boundary tensors and the shapes (32 entries, least recently built evicted first)."""
    assert kind is None or kind in MASK_KINDS, f"unknown flex attention mask {kind!r}; expected one of {MASK_KINDS}"
    key = (kind, cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), cu_seqlens_q._version, total_q, total_k, max_seqlen_q, max_seqlen_k, causal, sliding_window)
    hit = _CACHE.get(key)
    if hit is not None:
        return hit
    dev = cu_seqlens_q.device
    if kind in ("causal", "full", "sliding_window"):
        bm = BlockMask(_one_document(total_q, dev), _one_document(total_k, dev), total_q, total_k, causal=(kind != "full") and causal, window=(sliding_window or None) if kind == "sliding_window" else None)
    elif kind == "document":
        bm = BlockMask(cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=causal, window=None)
    else:
        bm = BlockMask(cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=causal, window=sliding_window or None)
    _CACHE[key] = bm
    _CACHE_ORDER.append(key)
    if len(_CACHE_ORDER) > _CACHE_SIZE:
        _CACHE.pop(_CACHE_ORDER.pop(0), None)
    return bm


@functools.lru_cache(maxsize=32)
def create_block_mask_cached(kind: str, total_q: int, total_k: int, sliding_window: Optional[int] = None, device: str = "cpu") -> BlockMask:
    """Document-free masks by shape (same role as the reference's ``create_block_mask_cached``, nn/flex_attention.py:138-142)."""
    dev = torch.device(device)
    return BlockMask(_one_document(total_q, dev), _one_document(total_k, dev), total_q, total_k, causal=kind != "full", window=sliding_window if kind == "sliding_window" else None)


# ---------------------------------------------------------------------------- score modification
def softcapped_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: BlockMask, softcap: float, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Attention with ``softcap * tanh(score / softcap)`` applied to the scaled scores before masking (the score modifier of
    the reference, nn/flex_attention.py:12-34).  fp32 masked softmax per document: no kernel implements the cap."""
    import math

    Tq, Hq, D = q.shape
    rep = Hq // k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    cq, ck = mask.cu_seqlens_q.tolist(), mask.cu_seqlens_k.tolist()
    out = torch.zeros(Tq, Hq, D, dtype=torch.float32, device=q.device)
    for d in range(len(cq) - 1):
        lq, lk = cq[d + 1] - cq[d], ck[d + 1] - ck[d]
        if lq == 0 or lk == 0:
            continue
        qd = q[cq[d] : cq[d + 1]].float().transpose(0, 1)
        kd = k[ck[d] : ck[d + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vd = v[ck[d] : ck[d + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qd, kd.transpose(1, 2)) * scale
        s = softcap * torch.tanh(s / softcap)
        i = torch.arange(lq, device=q.device).unsqueeze(1) + (lk - lq)
        j = torch.arange(lk, device=q.device).unsqueeze(0)
        keep = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if mask.causal:
            keep &= j <= i
        if mask.window:
            keep &= j > i - mask.window
        p = torch.softmax(s.masked_fill(~keep, float("-inf")), dim=-1)
        out[cq[d] : cq[d + 1]] = torch.matmul(torch.nan_to_num(p, nan=0.0), vd).transpose(0, 1)
    return out.to(q.dtype)
