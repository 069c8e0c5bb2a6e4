"""Causal attention over a context-parallel group with zig-zag sequence sharding.

Each rank holds, for every batch row, chunks ``r`` and ``2*cp-1-r`` of the ``2*cp`` equal chunks of the sequence
(``zigzag.py``), so causal work is balanced (the reference's context parallelism slices contiguously, which leaves the
last rank with about cp times the work of the first: reference src/nanotron/nn/llama3_ring_attention.py:63-158).

Variant "allgather" (what every registry name maps to at the moment): K and V are all-gathered over the group with a
differentiable all-gather (its backward is the reduce-scatter of dK / dV), put back in global order, and each of the two
local query chunks attends the key prefix that ends with it.  With ``lq = c`` queries against ``lk = (i+1)*c`` keys the
bottom-right aligned causal mask of the attention kernels is exactly the global causal mask, so the ordinary
variable-length kernel does the work and no special masking is needed.

``merge_attention_states`` combines partial results (out, lse) over disjoint key sets; it is the building block of the
blockwise / ring schedule.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200 import ops
from nanotron_b200.parallel.context_parallel.zigzag import zigzag_chunk_ids


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


def ring_attention(q, k, v, cp_pg, causal: bool = True, softmax_scale: Optional[float] = None, variant: str = "allgather", position_ids: Optional[torch.Tensor] = None, **_):
    """q: [b*s_local, Hq, D]; k, v: [b*s_local, Hkv, D] with the local tokens of every batch row in zig-zag order
    (first chunk ``r``, then chunk ``2cp-1-r``).  ``position_ids`` [b, s_local] gives the batch size."""
    cp = cp_pg.size() if cp_pg is not None else 1
    assert position_ids is not None, "context-parallel attention needs position_ids to know the batch layout"
    b, s_local = position_ids.shape
    if cp == 1:
        cu = torch.arange(0, (b + 1) * s_local, s_local, dtype=torch.int32, device=q.device)
        return ops.flash_attn_varlen(q, k, v, cu, cu, s_local, s_local, causal=causal, softmax_scale=softmax_scale)
    assert causal, "zig-zag sharding is only meaningful for causal attention"
    if variant == "fused" or ops._ATTN == "native":
        from nanotron_b200.parallel.context_parallel import fused_ring

        if fused_ring.supported(q, k, cp_pg, s_local // 2):
            # K / V stay on their owners: the attention kernels read / reduce them over NVLink tile by tile
            return fused_ring.fused_ring_attention(q, k, v, cp_pg, batch=b, softmax_scale=softmax_scale)
        assert variant != "fused", "fused context-parallel attention needs CUDA, bf16, head_dim 128, chunks of a multiple of 128 tokens and cp <= 8 inside one node"
    rank = dist.get_rank(cp_pg)
    c = s_local // 2
    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    # gather K and V: [cp, b, 2, c, Hkv, D] -> global order [b, 2cp*c, Hkv, D]
    kv = torch.stack([k, v], dim=0).reshape(2, b, 2, c, Hkv, D)
    gathered = _AllGatherDim0.apply(kv.reshape(1, *kv.shape), cp_pg)  # [cp, 2, b, 2, c, Hkv, D]
    order = []
    for chunk in range(2 * cp):
        src = chunk if chunk < cp else 2 * cp - 1 - chunk
        order.append((src, 0 if chunk < cp else 1))
    glob = torch.stack([gathered[src, :, :, half] for src, half in order], dim=2)  # [2, b, 2cp, c, Hkv, D]
    glob = glob.reshape(2, b, 2 * cp * c, Hkv, D)
    qb = q.reshape(b, 2, c, Hq, D)
    outs = []
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
