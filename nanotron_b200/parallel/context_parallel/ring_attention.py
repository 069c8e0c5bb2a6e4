"""Causal attention over a context-parallel group with zig-zag sequence sharding.

Each rank holds, for every batch row, chunks ``r`` and ``2*cp-1-r`` of the ``2*cp`` equal chunks of the sequence
(``zigzag.py``), so causal work is balanced (the reference's context parallelism slices contiguously, which leaves the
last rank with about cp times the work of the first: reference src/nanotron/nn/llama3_ring_attention.py:63-158).

Variant "allgather" (registry name ``llama3_ring_attention``, the default): K and V are all-gathered over the group with a
differentiable all-gather (its backward is the reduce-scatter of dK / dV), put back in global order, and each of the two
local query chunks attends the key prefix that ends with it.  With ``lq = c`` queries against ``lk = (i+1)*c`` keys the
bottom-right aligned causal mask of the attention kernels is exactly the global causal mask, so the ordinary
variable-length kernel does the work and no special masking is needed.

Variant "ring" (registry names ``ring`` and ``ring_flash_triton``; capability parity: reference src/nanotron/nn/ring_attention.py,
ring_attention_lucidrain.py): K / V blocks travel around the group with send / recv, one hop per step, while the block that
has arrived is attended; memory per rank stays at two K / V blocks whatever the group size.  Under zig-zag sharding a step
needs no mask beyond "causal" for the rank's own block: a block from a lower rank is seen in its first half by all local
queries, a block from a higher rank is seen entirely by the second half of the local queries.  Partial results are merged
with their log-sum-exp; the backward runs the ring again with the final (out, lse), dK / dV travelling with their block.

Packed documents (``doc_masking``: a position id of 0 starts a document) are handled by the "allgather" variant: the position ids
are gathered once per micro-batch, every local query chunk is cut at the document starts inside it, and each piece attends the
keys from the start of its document up to its own end -- consecutive key ranges of the gathered K / V, so this is again one call
of the variable-length kernel per chunk (what the reference does for contiguous shards: src/nanotron/nn/llama3_ring_attention.py:10-60).

``merge_attention_states`` combines partial results (out, lse) over disjoint key sets; it is the building block of the
blockwise / ring schedule.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200 import ops
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel.context_parallel.zigzag import zigzag_chunk_ids

_logger = get_logger(__name__)


class _AllGatherDim0(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = x.new_empty((group.size() * x.shape[0], *x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        g = g.contiguous()
        out = g.new_empty((g.shape[0] // group.size(), *g.shape[1:]))
        dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=group)
        return out, None


def merge_attention_states(out_a: torch.Tensor, lse_a: torch.Tensor, out_b: torch.Tensor, lse_b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """out: [T, H, D], lse: [H, T].  Softmax-weighted combination of two partial attentions over disjoint key sets."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).transpose(0, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).transpose(0, 1).unsqueeze(-1)
    wa = torch.nan_to_num(wa, nan=0.0)
    wb = torch.nan_to_num(wb, nan=0.0)
    return (out_a.float() * wa + out_b.float() * wb).to(out_a.dtype), lse


def _use_native(q, k, v) -> bool:
    if not q.is_cuda or ops.get_mode() == "torch" or ops._ATTN == "sdpa":
        return False
    from nanotron_b200.ops import native

    return native.flash_attn_supported(q, k, v, None)


def _cu(b: int, n: int, device) -> torch.Tensor:
    return torch.arange(0, (b + 1) * n, n, dtype=torch.int32, device=device)


def _block_fwd(q, k, v, b: int, causal: bool, scale: float):
    """One block of the ring: q [b*lq, Hq, D] against k, v [b*lk, Hkv, D] (b equal-length rows).  Returns out [b*lq, Hq, D]
    and lse [Hq, b*lq] (fp32).  In-tree kernel on CUDA, fp32 matrix math elsewhere."""
    lq, lk = q.shape[0] // b, k.shape[0] // b
    if _use_native(q, k, v):
        from nanotron_b200.ops import native

        return native.flash_attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), _cu(b, lq, q.device), _cu(b, lk, q.device), lq, lk, causal, scale, None)
    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    g = Hq // Hkv
    acc = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf = q.to(acc).reshape(b, lq, Hkv, g, D)
    kf, vf = k.to(acc).reshape(b, lk, Hkv, D), v.to(acc).reshape(b, lk, Hkv, D)
    s = torch.einsum("bqhgd,bkhd->bhgqk", qf, kf) * scale
    if causal:
        keep = torch.ones(lq, lk, dtype=torch.bool, device=q.device).tril(diagonal=lk - lq)
        s = s.masked_fill(~keep, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)  # [b, Hkv, g, lq]
    p = torch.exp(s - lse.unsqueeze(-1))
    out = torch.einsum("bhgqk,bkhd->bqhgd", p, vf).reshape(b * lq, Hq, D)
    return out.to(q.dtype), lse.permute(1, 2, 0, 3).reshape(Hq, b * lq).to(torch.float32 if acc == torch.float32 else acc)


def _block_bwd(dout, q, k, v, out, lse, b: int, causal: bool, scale: float):
    """Gradients of one block given the FINAL out and lse of the whole attention (probabilities exp(s - lse) are then the
    global ones, so the blocks' dQ simply add up).  Returns dq, dk, dv in fp32 (fp64 for fp64 inputs)."""
    lq, lk = q.shape[0] // b, k.shape[0] // b
    if _use_native(q, k, v):
        from nanotron_b200.ops import native

        dq, dk, dv = native.flash_attn_bwd(dout.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous(), lse.contiguous(), _cu(b, lq, q.device),
                                           _cu(b, lk, q.device), lq, lk, causal, scale, None)
        return dq.float(), dk.float(), dv.float()
    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    g = Hq // Hkv
    acc = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf = q.to(acc).reshape(b, lq, Hkv, g, D)
    kf, vf = k.to(acc).reshape(b, lk, Hkv, D), v.to(acc).reshape(b, lk, Hkv, D)
    do = dout.to(acc).reshape(b, lq, Hkv, g, D)
    of = out.to(acc).reshape(b, lq, Hkv, g, D)
    s = torch.einsum("bqhgd,bkhd->bhgqk", qf, kf) * scale
    if causal:
        keep = torch.ones(lq, lk, dtype=torch.bool, device=q.device).tril(diagonal=lk - lq)
        s = s.masked_fill(~keep, float("-inf"))
    l = lse.to(acc).reshape(Hkv, g, b, lq).permute(2, 0, 1, 3)  # [b, Hkv, g, lq]
    p = torch.exp(s - l.unsqueeze(-1))
    dv = torch.einsum("bhgqk,bqhgd->bkhd", p, do)
    dp = torch.einsum("bqhgd,bkhd->bhgqk", do, vf)
    delta = (do * of).sum(-1).permute(0, 2, 3, 1)  # [b, Hkv, g, lq]
    ds = p * (dp - delta.unsqueeze(-1)) * scale
    dq = torch.einsum("bhgqk,bkhd->bqhgd", ds, kf).reshape(b * lq, Hq, D)
    dk = torch.einsum("bhgqk,bqhgd->bkhd", ds, qf)
    return dq, dk.reshape(b * lk, Hkv, D), dv.reshape(b * lk, Hkv, D)


def _ring_exchange(send: torch.Tensor, recv: torch.Tensor, group):
    """Posts `send` to the next rank of the group and `recv` from the previous one; returns the requests."""
    n, me = group.size(), dist.get_rank(group)
    nxt, prv = dist.get_global_rank(group, (me + 1) % n), dist.get_global_rank(group, (me - 1) % n)
    ops_ = [torch.distributed.P2POp(torch.distributed.isend, send, nxt, group), torch.distributed.P2POp(torch.distributed.irecv, recv, prv, group)]
    return torch.distributed.batch_isend_irecv(ops_)


def _half(t: torch.Tensor, b: int, which: int, token_dim: int = 0) -> torch.Tensor:
    """Rows of the first / second local chunk of every batch row (tokens are laid out [b, 2, c] along `token_dim`)."""
    shape = list(t.shape)
    n = shape[token_dim]
    view = t.reshape(*shape[:token_dim], b, 2, n // (2 * b), *shape[token_dim + 1 :])
    return view.select(token_dim + 1, which).reshape(*shape[:token_dim], n // 2, *shape[token_dim + 1 :])


class _ZigZagRing(torch.autograd.Function):
    """Causal attention over zig-zag shards with K / V travelling around the group (see the module docstring)."""

    @staticmethod
    def forward(ctx, q, k, v, group, b, scale):
        cp, rank = group.size(), dist.get_rank(group)
        cur = torch.stack([k, v], dim=0).contiguous()  # [2, b*2c, Hkv, D]
        out = lse = None
        for step in range(cp):
            reqs, nxt = [], None
            if step + 1 < cp:
                nxt = torch.empty_like(cur)
                reqs = _ring_exchange(cur, nxt, group)  # in flight while this block is attended
            src = (rank - step) % cp
            if step == 0:
                o, l = _block_fwd(q, cur[0], cur[1], b, True, scale)
                out, lse = o.to(torch.float64 if o.dtype == torch.float64 else torch.float32), l
            elif src < rank:
                # an earlier rank's block: its first chunk precedes both local chunks, its second follows both
                o, l = _block_fwd(q, _half(cur[0], b, 0), _half(cur[1], b, 0), b, False, scale)
                out, lse = _merge_into(out, lse, o, l)
            else:
                # a later rank's block: both of its chunks lie between the two local chunks
                o, l = _block_fwd(_half(q, b, 1), cur[0], cur[1], b, False, scale)
                Hq = q.shape[1]
                o2, l2 = _merge_into(_half(out, b, 1), _half(lse, b, 1, token_dim=1), o, l)
                out = out.clone()
                lse = lse.clone()
                out.reshape(b, 2, -1, Hq, q.shape[2])[:, 1] = o2.reshape(b, -1, Hq, q.shape[2])
                lse.reshape(Hq, b, 2, -1)[:, :, 1] = l2.reshape(Hq, b, -1)
            for r in reqs:
                r.wait()
            if nxt is not None:
                cur = nxt
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.group, ctx.b, ctx.scale = group, b, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, b, scale = ctx.group, ctx.b, ctx.scale
        cp, rank = group.size(), dist.get_rank(group)
        acc = torch.float64 if q.dtype == torch.float64 else torch.float32
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=acc, device=q.device)
        cur = torch.stack([k, v], dim=0).contiguous()
        dcur = torch.zeros(cur.shape, dtype=acc, device=q.device)  # gradient of the block in hand, summed over the ranks it has visited
        for step in range(cp):
            reqs, nxt = [], None
            if step + 1 < cp:
                nxt = torch.empty_like(cur)
                reqs = _ring_exchange(cur, nxt, group)
            src = (rank - step) % cp
            if step == 0:
                g_q, g_k, g_v = _block_bwd(dout, q, cur[0], cur[1], out, lse, b, True, scale)
                dq += g_q
                dcur[0] += g_k
                dcur[1] += g_v
            elif src < rank:
                g_q, g_k, g_v = _block_bwd(dout, q, _half(cur[0], b, 0), _half(cur[1], b, 0), out, lse, b, False, scale)
                dq += g_q
                Hkv, D = k.shape[1], k.shape[2]
                dcur[0].reshape(b, 2, -1, Hkv, D)[:, 0] += g_k.reshape(b, -1, Hkv, D)
                dcur[1].reshape(b, 2, -1, Hkv, D)[:, 0] += g_v.reshape(b, -1, Hkv, D)
            else:
                g_q, g_k, g_v = _block_bwd(_half(dout, b, 1), _half(q, b, 1), cur[0], cur[1], _half(out, b, 1), _half(lse, b, 1, token_dim=1), b, False, scale)
                Hq, D = q.shape[1], q.shape[2]
                dq.reshape(b, 2, -1, Hq, D)[:, 1] += g_q.reshape(b, -1, Hq, D)
                dcur[0] += g_k
                dcur[1] += g_v
            for r in reqs:
                r.wait()
            # the block's gradient follows the block; after the last step this hop brings it home
            dnxt = torch.empty_like(dcur)
            for r in _ring_exchange(dcur, dnxt, group):
                r.wait()
            dcur = dnxt
            if nxt is not None:
                cur = nxt
        return dq.to(q.dtype), dcur[0].to(k.dtype), dcur[1].to(v.dtype), None, None, None


def _merge_into(out, lse, o, l):
    """(out fp32 [T, H, D], lse [H, T]) merged with another partial result over a disjoint key set."""
    new = torch.logaddexp(lse, l.to(lse.dtype))
    wa = torch.exp(lse - new).transpose(0, 1).unsqueeze(-1)
    wb = torch.exp(l.to(lse.dtype) - new).transpose(0, 1).unsqueeze(-1)
    return out * wa.to(out.dtype) + o.to(out.dtype) * wb.to(out.dtype), new


def _global_order(cp: int):
    """(source rank, half) of the 2cp chunks in global order: chunk i < cp is the first half of rank i, chunk i >= cp the second
    half of rank 2cp-1-i."""
    return [(chunk, 0) if chunk < cp else (2 * cp - 1 - chunk, 1) for chunk in range(2 * cp)]


def _document_plan(position_ids: torch.Tensor, cp_pg, rank: int, cp: int, c: int):
    """For each of the two local query chunks: (query piece lengths, key range lengths, per row (first key, end key)).

    A piece is a run of queries of one document inside the chunk; its keys start where its document starts (possibly in an
    earlier chunk, on another rank) and end with the piece.  The plan depends on the micro-batch only, so it is computed by the
    first layer that asks and reused by the others (one small all-gather and one device -> host copy per micro-batch)."""
    # cached on the tensor object itself: the decoder layers of a stage hand the same object on, and a later micro-batch is a new
    # object even when the allocator gives it the same address
    cached = getattr(position_ids, "_ntb_document_plan", None)
    if cached is not None and cached[0] == (position_ids._version, rank, cp, c):
        return cached[1]
    b = position_ids.shape[0]
    local = position_ids.reshape(1, b, 2, c).contiguous()
    gathered = local.new_empty((cp, b, 2, c))
    dist.all_gather_into_tensor(gathered, local, group=cp_pg)
    glob = torch.stack([gathered[src, :, half] for src, half in _global_order(cp)], dim=1).reshape(b, 2 * cp * c)
    starts = (glob == 0).cpu()
    starts[:, 0] = True  # a row may begin in the middle of a document
    plan = []
    for chunk in zigzag_chunk_ids(rank, cp):
        lo, hi = chunk * c, (chunk + 1) * c
        q_lens, k_lens, k_ranges = [], [], []
        for row in range(b):
            doc_starts = torch.nonzero(starts[row, :hi]).flatten().tolist()
            first = max(s for s in doc_starts if s <= lo)
            bounds = [lo] + [s for s in doc_starts if lo < s] + [hi]
            for j in range(len(bounds) - 1):
                q_lens.append(bounds[j + 1] - bounds[j])
                k_lens.append(bounds[j + 1] - (first if j == 0 else bounds[j]))
            k_ranges.append((first, hi))
        plan.append((q_lens, k_lens, k_ranges))
    position_ids._ntb_document_plan = ((position_ids._version, rank, cp, c), plan)
    return plan


def _cumulative(lengths, device) -> torch.Tensor:
    return torch.tensor([0] + lengths, dtype=torch.int64).cumsum(0).to(torch.int32).to(device)


def ring_attention(q, k, v, cp_pg, causal: bool = True, softmax_scale: Optional[float] = None, variant: str = "allgather", position_ids: Optional[torch.Tensor] = None,
                   doc_masking: bool = False, **_):
    """q: [b*s_local, Hq, D]; k, v: [b*s_local, Hkv, D] with the local tokens of every batch row in zig-zag order
    (first chunk ``r``, then chunk ``2cp-1-r``).  ``position_ids`` [b, s_local] gives the batch size and, with ``doc_masking``,
    the document starts (position 0): attention then stays inside a document."""
    cp = cp_pg.size() if cp_pg is not None else 1
    assert position_ids is not None, "context-parallel attention needs position_ids to know the batch layout"
    b, s_local = position_ids.shape
    if cp == 1:
        cu = torch.arange(0, (b + 1) * s_local, s_local, dtype=torch.int32, device=q.device)
        return ops.flash_attn_varlen(q, k, v, cu, cu, s_local, s_local, causal=causal, softmax_scale=softmax_scale)
    assert causal, "zig-zag sharding is only meaningful for causal attention"
    if doc_masking and variant != "allgather":
        from nanotron_b200.logging import warn_once

        warn_once(logger=_logger, msg=f"context-parallel attention variant {variant!r} has no document masking: packed documents use the all-gather variant", rank=0)
        variant = "allgather"
    if not doc_masking and (variant == "fused" or ops._ATTN == "native"):
        from nanotron_b200.parallel.context_parallel import fused_ring

        if fused_ring.supported(q, k, cp_pg, s_local // 2):
            # K / V stay on their owners: the attention kernels read / reduce them over NVLink tile by tile
            return fused_ring.fused_ring_attention(q, k, v, cp_pg, batch=b, softmax_scale=softmax_scale)
        assert variant != "fused", "fused context-parallel attention needs CUDA, bf16, head_dim 128, chunks of a multiple of 128 tokens and cp <= 8 inside one node"
    if variant == "ring":
        scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
        return _ZigZagRing.apply(q.contiguous(), k.contiguous(), v.contiguous(), cp_pg, b, scale)
    rank = dist.get_rank(cp_pg)
    c = s_local // 2
    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    # gather K and V: [cp, b, 2, c, Hkv, D] -> global order [b, 2cp*c, Hkv, D]
    kv = torch.stack([k, v], dim=0).reshape(2, b, 2, c, Hkv, D)
    gathered = _AllGatherDim0.apply(kv.reshape(1, *kv.shape), cp_pg)  # [cp, 2, b, 2, c, Hkv, D]
    glob = torch.stack([gathered[src, :, :, half] for src, half in _global_order(cp)], dim=2)  # [2, b, 2cp, c, Hkv, D]
    glob = glob.reshape(2, b, 2 * cp * c, Hkv, D)
    qb = q.reshape(b, 2, c, Hq, D)
    outs = []
    if doc_masking:
        for half, (q_lens, k_lens, k_ranges) in enumerate(_document_plan(position_ids, cp_pg, rank, cp, c)):
            qh = qb[:, half].reshape(b * c, Hq, D)
            kh = torch.cat([glob[0, row, first:end] for row, (first, end) in enumerate(k_ranges)])
            vh = torch.cat([glob[1, row, first:end] for row, (first, end) in enumerate(k_ranges)])
            o = ops.flash_attn_varlen(qh, kh, vh, _cumulative(q_lens, q.device), _cumulative(k_lens, q.device), max(q_lens), max(k_lens), causal=True, softmax_scale=softmax_scale)
            outs.append(o.reshape(b, c, Hq, D))
        return torch.stack(outs, dim=1).reshape(b * s_local, Hq, D)
    for half, chunk in enumerate(zigzag_chunk_ids(rank, cp)):
        lk = (chunk + 1) * c
        qh = qb[:, half].reshape(b * c, Hq, D)
        kh = glob[0, :, :lk].reshape(b * lk, Hkv, D)
        vh = glob[1, :, :lk].reshape(b * lk, Hkv, D)
        cu_q = torch.arange(0, (b + 1) * c, c, dtype=torch.int32, device=q.device)
        cu_k = torch.arange(0, (b + 1) * lk, lk, dtype=torch.int32, device=q.device)
        o = ops.flash_attn_varlen(qh, kh, vh, cu_q, cu_k, c, lk, causal=True, softmax_scale=softmax_scale)
        outs.append(o.reshape(b, c, Hq, D))
    return torch.stack(outs, dim=1).reshape(b * s_local, Hq, D)
