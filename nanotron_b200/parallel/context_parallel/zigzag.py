"""Zig-zag sequence sharding for causal context parallelism.

The sequence is cut into ``2*cp`` equal chunks; rank r owns chunks ``r`` and ``2*cp-1-r``.  Under a causal mask this
gives every rank the same amount of attention work (an early cheap chunk plus a late expensive one), unlike
contiguous slicing where the last rank does about cp times the work of the first.
"""
from __future__ import annotations

import torch


def zigzag_chunk_ids(cp_rank: int, cp_size: int):
    return cp_rank, 2 * cp_size - 1 - cp_rank


def zigzag_slice(x: torch.Tensor, cp_rank: int, cp_size: int, dim: int = 1) -> torch.Tensor:
    """Local part of ``x`` along ``dim`` (length must be divisible by 2*cp)."""
    if cp_size == 1:
        return x
    n = x.shape[dim]
    assert n % (2 * cp_size) == 0, f"sequence length {n} must be divisible by 2*cp={2 * cp_size}"
    c = n // (2 * cp_size)
    a, b = zigzag_chunk_ids(cp_rank, cp_size)
    return torch.cat([x.narrow(dim, a * c, c), x.narrow(dim, b * c, c)], dim=dim)


def zigzag_positions(seq_len: int, cp_rank: int, cp_size: int, device=None) -> torch.Tensor:
    """Global positions of the tokens held by ``cp_rank``."""
    if cp_size == 1:
        return torch.arange(seq_len, device=device)
    c = seq_len // (2 * cp_size)
    a, b = zigzag_chunk_ids(cp_rank, cp_size)
    return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])


def zigzag_unshard(parts, dim: int = 1) -> torch.Tensor:
    """Inverse of ``zigzag_slice``: ``parts[r]`` is rank r's local tensor."""
    cp = len(parts)
    if cp == 1:
        return parts[0]
    chunks = [None] * (2 * cp)
    for r, p in enumerate(parts):
        a, b = zigzag_chunk_ids(r, cp)
        first, second = p.chunk(2, dim=dim)
        chunks[a], chunks[b] = first, second
    return torch.cat(chunks, dim=dim)
