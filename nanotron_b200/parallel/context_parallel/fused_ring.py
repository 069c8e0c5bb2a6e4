"""Context-parallel causal attention with the key / value exchange inside the attention kernel.

Every rank publishes its K and V (zig-zag layout: chunk ``r`` then chunk ``2 cp - 1 - r`` of every batch row) in peer-mapped buffers;
the tcgen05 flash-attention kernels then read the key tiles they need straight from their owners over NVLink (forward) and add the
dK / dV contributions of the local queries into the owners' fp32 accumulators (backward) -- see ``ops/csrc/attention_fwd.cu`` and
``attention_bwd.cu``.  There is no all-gather, no ring of NCCL send / recv and no host-side merging of partial softmax states.
(The reference's context parallelism, src/nanotron/nn/llama3_ring_attention.py, all-gathers K / V with NCCL and calls flash-attn per
chunk; its ring variants exchange KV blocks with batched isend / irecv between kernel launches.)

Cross-rank ordering uses the device barrier of ``parallel.symm`` (bounded waits):
  forward : copy K, V -> barrier -> kernel -> barrier (buffers may be overwritten by the next call)
  backward: copy K, V, zero the accumulators -> barrier -> kernel -> barrier -> cast this rank's accumulators to bf16
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Dict, Optional, Tuple

import torch

from nanotron_b200 import distributed as dist

_CONTEXTS: Dict[Tuple[int, int, int, int], "FusedCPContext"] = {}
_DECLARED = False
HEAD_DIM = 128


def _lib():
    global _DECLARED
    from nanotron_b200.ops import native

    L = native.lib()
    if not _DECLARED:
        L.ntb_flash_attn_fwd_cp.restype = c_int
        L.ntb_flash_attn_fwd_cp.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_int64] * 4 + [c_float, c_void_p, c_void_p]
        if hasattr(L, "ntb_flash_attn_fwd2_cp"):  # two query tiles per CTA (ops/csrc/attention_fwd2.cu), same contract
            L.ntb_flash_attn_fwd2_cp.restype = c_int
            L.ntb_flash_attn_fwd2_cp.argtypes = L.ntb_flash_attn_fwd_cp.argtypes
        L.ntb_flash_attn_bwd_cp.restype = c_int
        L.ntb_flash_attn_bwd_cp.argtypes = [c_void_p] * 11 + [c_int] * 6 + [c_int64] * 5 + [c_float, c_void_p, c_void_p]
        L.ntb_cast_f32_to_bf16_rows.restype = c_int
        L.ntb_cast_f32_to_bf16_rows.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p]
        _DECLARED = True
    return L


class FusedCPContext:
    """Peer-mapped K / V buffers and dK / dV accumulators of one context-parallel group, for one (tokens, kv heads) shape."""

    def __init__(self, group, tokens: int, kv_heads: int):
        from nanotron_b200.parallel.symm import SymmetricAllocator

        self.group = group
        self.world = group.size()
        self.rank = dist.get_rank(group)
        self.tokens, self.kv_heads = tokens, kv_heads
        self.alloc = SymmetricAllocator(group)
        n = tokens * kv_heads * HEAD_DIM
        self.k = self.alloc.zeros(n, torch.bfloat16)
        self.v = self.alloc.zeros(n, torch.bfloat16)
        self.dk_acc = self.alloc.zeros(n, torch.float32)
        self.dv_acc = self.alloc.zeros(n, torch.float32)
        self.calls = 0

    def publish(self, k: torch.Tensor, v: torch.Tensor, zero_acc: bool):
        self.k.tensor.view(self.tokens, self.kv_heads, HEAD_DIM).copy_(k)
        self.v.tensor.view(self.tokens, self.kv_heads, HEAD_DIM).copy_(v)
        if zero_acc:
            self.dk_acc.tensor.zero_()
            self.dv_acc.tensor.zero_()
        self.alloc.barrier()


def supported(q: torch.Tensor, k: torch.Tensor, cp_pg, chunk: int) -> bool:
    from nanotron_b200 import ops
    from nanotron_b200.ops import native
    from nanotron_b200.parallel import symm

    return (
        q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == HEAD_DIM and chunk % 128 == 0 and cp_pg is not None and 1 < cp_pg.size() <= 8
        and ops.get_mode() != "torch" and native.available() and hasattr(native.lib(), "ntb_flash_attn_fwd_cp") and symm.is_available(cp_pg)
    )


def get_context(group, tokens: int, kv_heads: int) -> FusedCPContext:
    key = (id(group), tokens, kv_heads, torch.cuda.current_device())
    if key not in _CONTEXTS:
        _CONTEXTS[key] = FusedCPContext(group, tokens, kv_heads)
    return _CONTEXTS[key]


class _FusedCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cctx: FusedCPContext, batch: int, chunk: int, scale: float):
        from nanotron_b200.ops import native, native_gemm

        L = _lib()
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        q = q.contiguous()
        cctx.publish(k, v, zero_acc=False)
        out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        status = native_gemm.status_word(q.device)
        from nanotron_b200.ops import native_attn

        fwd = L.ntb_flash_attn_fwd2_cp if (hasattr(L, "ntb_flash_attn_fwd2_cp") and native_attn.FWD_VARIANT["kernel"] == "two_tile") else L.ntb_flash_attn_fwd_cp
        rc = fwd(q.data_ptr(), cctx.k.ptrs, cctx.v.ptrs, out.data_ptr(), lse.data_ptr(), batch, chunk, cctx.world, cctx.rank, Hq, Hkv,
                                     q.stride(0), q.stride(1), Hkv * D, D, scale, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "flash_attn_fwd_cp")
        cctx.alloc.barrier()  # every rank has finished reading K / V: the buffers may be reused
        cctx.calls += 1
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cctx, ctx.batch, ctx.chunk, ctx.scale = cctx, batch, chunk, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        from nanotron_b200.ops import native, native_gemm

        L = _lib()
        q, k, v, out, lse = ctx.saved_tensors
        cctx: FusedCPContext = ctx.cctx
        T, Hq, D = q.shape
        Hkv = k.shape[1]
        dout = dout.contiguous()
        cctx.publish(k, v, zero_acc=True)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
        dq_acc = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
        dq = torch.empty_like(q)
        status = native_gemm.status_word(q.device)
        stream = torch.cuda.current_stream().cuda_stream
        rc = L.ntb_flash_attn_bwd_cp(dout.data_ptr(), q.data_ptr(), cctx.k.ptrs, cctx.v.ptrs, out.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
                                     dq.data_ptr(), cctx.dk_acc.ptrs, cctx.dv_acc.ptrs, ctx.batch, ctx.chunk, cctx.world, cctx.rank, Hq, Hkv,
                                     q.stride(0), q.stride(1), Hkv * D, D, Hq * D, ctx.scale, status.data_ptr(), stream)
        native._check(rc, "flash_attn_bwd_cp")
        cctx.alloc.barrier()  # every rank's contributions to my dK / dV have landed
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
        for acc, dst in ((cctx.dk_acc, dk), (cctx.dv_acc, dv)):
            native._check(L.ntb_cast_f32_to_bf16_rows(acc.tensor.data_ptr(), dst.data_ptr(), T, Hkv, Hkv * D, stream), "cast_f32_to_bf16_rows")
        return dq, dk, dv, None, None, None, None


def fused_ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cp_pg, batch: int, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """q: [batch * s_local, Hq, 128]; k, v: [batch * s_local, Hkv, 128]; s_local = 2 chunks in zig-zag order.  Causal."""
    T = q.shape[0]
    chunk = T // batch // 2
    scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
    cctx = get_context(cp_pg, T, k.shape[1])
    return _FusedCPAttention.apply(q, k, v, cctx, batch, chunk, float(scale))
