"""ctypes bindings of ``libntb_kernels.so`` (the in-tree sm_100a kernels).

Every wrapper takes torch tensors, checks device / dtype / contiguity on the host, passes raw pointers plus the
current CUDA stream, and raises on a non-zero status.  The library is loaded lazily and only from the package
directory; on a machine with a GPU a missing library is an error (there is no silent PyTorch fallback for CUDA
tensors).  Outputs are allocated here with torch so they take part in the caching allocator and stream semantics.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path
from typing import List, Optional, Tuple

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent / "libntb_kernels.so"
_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class NativeKernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            raise NativeKernelError(f"{_LIB_PATH} is missing: run `python -m nanotron_b200.ops.build` (CUDA tensors never fall back to PyTorch ops)")
        _LIB = ctypes.CDLL(str(_LIB_PATH))
        _declare(_LIB)
    return _LIB


def available() -> bool:
    return _LIB_PATH.exists()


def _declare(L):
    L.ntb_norm_bwd_num_partials.restype = c_int
    L.ntb_norm_bwd_num_partials.argtypes = [c_int]
    L.ntb_norm_fwd.argtypes = [c_int, c_int] + [c_void_p] * 8 + [c_int, c_int, c_float, c_void_p]
    L.ntb_norm_bwd.argtypes = [c_int, c_int] + [c_void_p] * 11 + [c_int, c_int, c_void_p]
    L.ntb_rope.argtypes = [c_int] + [c_void_p] * 5 + [c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]
    L.ntb_swiglu_fwd.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p]
    L.ntb_swiglu_bwd.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
    L.ntb_ce_partials.argtypes = [c_int] + [c_void_p] * 5 + [c_int64, c_int, c_int64, c_void_p]
    L.ntb_ce_backward.argtypes = [c_int] + [c_void_p] * 6 + [c_int64, c_int, c_int64, c_void_p]
    L.ntb_adamw_flat.argtypes = [c_void_p] * 5 + [c_int64] + [c_void_p] * 3 + [c_int] + [c_float] * 5 + [c_void_p, c_void_p]
    L.ntb_sumsq_num_partials.restype = c_int
    L.ntb_sumsq.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p]
    if hasattr(L, "ntb_symm_barrier"):
        c_uint32, c_ull = ctypes.c_uint32, ctypes.c_ulonglong
        L.ntb_comm_max_ranks.restype = c_int
        L.ntb_dp_num_partials.restype = c_int
        L.ntb_symm_barrier.restype = c_int
        L.ntb_symm_barrier.argtypes = [c_void_p, c_int, c_int, c_uint32, c_ull, c_void_p, c_void_p]
        L.ntb_dp_reduce_scatter.restype = c_int
        L.ntb_dp_reduce_scatter.argtypes = [c_void_p, c_int, c_int, c_int64, c_int64, c_float, c_int, c_void_p, c_void_p, c_void_p]
        if hasattr(L, "ntb_dp_reduce_scatter_range"):
            L.ntb_dp_reduce_scatter_range.restype = c_int
            L.ntb_dp_reduce_scatter_range.argtypes = [c_void_p, c_int, c_int, c_int64, c_int64, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p]
        L.ntb_symm_wait.restype = c_int
        L.ntb_symm_wait.argtypes = [c_void_p, c_int, c_uint32, c_ull, c_void_p, c_void_p]
        if hasattr(L, "ntb_gemm_bf16_ag"):
            L.ntb_tp_allgather_push.restype = c_int
            L.ntb_tp_allgather_push.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_longlong, c_uint32, c_void_p, c_void_p]
            L.ntb_gemm_bf16_ag.restype = c_int
            L.ntb_gemm_bf16_ag.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_uint32, c_void_p, c_int, c_void_p]
            L.ntb_gemm_bf16_rs.restype = c_int
            L.ntb_gemm_bf16_rs.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_uint32, c_void_p, c_void_p, c_int, c_void_p]
            if hasattr(L, "ntb_gemm2_bf16_ag"):
                L.ntb_gemm2_bf16_ag.restype = c_int
                L.ntb_gemm2_bf16_ag.argtypes = L.ntb_gemm_bf16_ag.argtypes
                if hasattr(L, "ntb_gemm2_bf16_ag_local"):
                    a = L.ntb_gemm_bf16_ag.argtypes
                    L.ntb_gemm2_bf16_ag_local.restype = c_int
                    L.ntb_gemm2_bf16_ag_local.argtypes = [a[0], c_void_p, c_int64] + list(a[1:])
                L.ntb_gemm2_bf16_rs.restype = c_int
                L.ntb_gemm2_bf16_rs.argtypes = L.ntb_gemm_bf16_rs.argtypes
            L.ntb_tp_reduce_slots.restype = c_int
            L.ntb_tp_reduce_slots.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.c_longlong, c_uint32, c_ull, c_void_p, c_void_p]
        L.ntb_dp_adamw_allgather.restype = c_int
        L.ntb_dp_adamw_allgather.argtypes = [c_void_p] * 5 + [c_int, c_int, c_int64, c_int64] + [c_void_p] * 3 + [c_int] + [c_float] * 5 + [c_void_p, c_void_p]
    for fn in ("ntb_norm_fwd", "ntb_norm_bwd", "ntb_rope", "ntb_swiglu_fwd", "ntb_swiglu_bwd", "ntb_ce_partials", "ntb_ce_backward", "ntb_adamw_flat", "ntb_sumsq"):
        getattr(L, fn).restype = c_int
    from nanotron_b200.ops import native_gemm, native_attn  # noqa: F401  (declare their symbols when present)

    native_gemm.declare(L)
    native_attn.declare(L)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str):
    from nanotron_b200.ops import LAUNCH_COUNTER

    LAUNCH_COUNTER["n"] += 1
    if rc != 0:
        detail = {1: "unsupported shape or alignment", 2: "CUDA launch error", 3: "device-side wait timed out"}.get(rc, "unknown")
        raise NativeKernelError(f"{what} failed with status {rc} ({detail})")


# ---------------------------------------------------------------------------- norms
def rmsnorm_fwd(x2, r2, weight, eps):
    assert x2.is_contiguous() and weight.is_contiguous() and x2.dtype == weight.dtype
    rows, cols = x2.shape
    y = torch.empty_like(x2)
    pre = torch.empty_like(x2) if r2 is not None else x2
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        rc = lib().ntb_norm_fwd(1, _DT[x2.dtype], x2.data_ptr(), _ptr(r2), weight.data_ptr(), None, y.data_ptr(), pre.data_ptr() if r2 is not None else None, None, rstd.data_ptr(), rows, cols, float(eps), _stream(x2))
    _check(rc, "rmsnorm_fwd")
    return y, pre, rstd


def rmsnorm_bwd(dy2, pre, weight, rstd, dres):
    rows, cols = dy2.shape
    L = lib()
    nparts = L.ntb_norm_bwd_num_partials(rows)
    dx = torch.empty_like(pre)
    partial = torch.empty((nparts, cols), dtype=torch.float32, device=dy2.device)
    dw = torch.empty(cols, dtype=torch.float32, device=dy2.device)
    with torch.cuda.device(dy2.device):
        rc = L.ntb_norm_bwd(1, _DT[dy2.dtype], dy2.data_ptr(), pre.data_ptr(), weight.data_ptr(), None, rstd.data_ptr(), _ptr(dres), dx.data_ptr(), partial.data_ptr(), None, dw.data_ptr(), None, rows, cols, _stream(dy2))
    _check(rc, "rmsnorm_bwd")
    return dx, dw


def layernorm_fwd(x2, r2, weight, bias, eps):
    rows, cols = x2.shape
    y = torch.empty_like(x2)
    pre = torch.empty_like(x2) if r2 is not None else x2
    mean = torch.empty(rows, dtype=torch.float32, device=x2.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    with torch.cuda.device(x2.device):
        rc = lib().ntb_norm_fwd(0, _DT[x2.dtype], x2.data_ptr(), _ptr(r2), weight.data_ptr(), _ptr(bias), y.data_ptr(), pre.data_ptr() if r2 is not None else None, mean.data_ptr(), rstd.data_ptr(), rows, cols, float(eps), _stream(x2))
    _check(rc, "layernorm_fwd")
    return y, pre, mean, rstd


def layernorm_bwd(dy2, pre, weight, mean, rstd, dres, has_bias):
    rows, cols = dy2.shape
    L = lib()
    nparts = L.ntb_norm_bwd_num_partials(rows)
    dx = torch.empty_like(pre)
    partial = torch.empty((2, nparts, cols), dtype=torch.float32, device=dy2.device)
    dw = torch.empty(cols, dtype=torch.float32, device=dy2.device)
    db = torch.empty(cols, dtype=torch.float32, device=dy2.device)
    with torch.cuda.device(dy2.device):
        rc = L.ntb_norm_bwd(0, _DT[dy2.dtype], dy2.data_ptr(), pre.data_ptr(), weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _ptr(dres), dx.data_ptr(), partial[0].data_ptr(), partial[1].data_ptr(), dw.data_ptr(), db.data_ptr(), rows, cols, _stream(dy2))
    _check(rc, "layernorm_bwd")
    return dx, dw, (db if has_bias else None)


# ---------------------------------------------------------------------------- rope / swiglu
def rope(x, cos, sin, interleaved: bool, inverse: bool, inplace: bool, positions: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """x: [T, H, D] with contiguous last dim (any token / head strides that are multiples of 8 elements).  ``out`` may be a
    strided [T, H, D] view (e.g. a slice of a fused qkv gradient buffer)."""
    T, H, D = x.shape
    assert x.stride(-1) == 1 and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    if out is None:
        out = x if inplace else torch.empty((T, H, D), dtype=x.dtype, device=x.device)
    else:
        assert out.shape == x.shape and out.dtype == x.dtype and out.stride(-1) == 1
    if positions is not None:
        positions = positions.to(torch.int64).contiguous()
    with torch.cuda.device(x.device):
        rc = lib().ntb_rope(_DT[x.dtype], x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), _ptr(positions), T, H, D, x.stride(0), x.stride(1), out.stride(0), out.stride(1), int(interleaved), int(inverse), _stream(x))
    _check(rc, "rope")
    return out


def swiglu_fwd(gate_up):
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * inter)
    out = torch.empty((*gate_up.shape[:-1], inter), dtype=gate_up.dtype, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        rc = lib().ntb_swiglu_fwd(_DT[gate_up.dtype], gate_up.data_ptr(), out.data_ptr(), rows, inter, _stream(gate_up))
    _check(rc, "swiglu_fwd")
    return out


def swiglu_bwd(gate_up, dout):
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * inter)
    dgu = torch.empty_like(gate_up)
    with torch.cuda.device(gate_up.device):
        rc = lib().ntb_swiglu_bwd(_DT[gate_up.dtype], gate_up.data_ptr(), dout.data_ptr(), dgu.data_ptr(), rows, inter, _stream(gate_up))
    _check(rc, "swiglu_bwd")
    return dgu


# ---------------------------------------------------------------------------- cross entropy
def ce_partials(logits2, target, vocab_start: int):
    rows, vocab = logits2.shape
    out = torch.empty((3, rows), dtype=torch.float32, device=logits2.device)
    target = target.to(torch.int64)
    with torch.cuda.device(logits2.device):
        rc = lib().ntb_ce_partials(_DT[logits2.dtype], logits2.data_ptr(), target.data_ptr(), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), rows, vocab, int(vocab_start), _stream(logits2))
    _check(rc, "ce_partials")
    return out[0], out[1], out[2]


def ce_backward(logits2, target, logz, grad_loss, grad_z, vocab_start: int, inplace: bool = True):
    rows, vocab = logits2.shape
    assert logits2.is_contiguous()
    grad = logits2 if inplace else torch.empty_like(logits2)
    target = target.to(torch.int64)
    grad_loss = grad_loss.contiguous().float()
    gz = grad_z.contiguous().float() if grad_z is not None else None
    with torch.cuda.device(logits2.device):
        rc = lib().ntb_ce_backward(_DT[logits2.dtype], logits2.data_ptr(), target.data_ptr(), logz.data_ptr(), grad_loss.data_ptr(), _ptr(gz), grad.data_ptr(), rows, vocab, int(vocab_start), _stream(logits2))
    _check(rc, "ce_backward")
    return grad


# ---------------------------------------------------------------------------- optimizer
def adamw_flat(p, g, m, v, p16, seg_end, seg_lr, seg_wd, beta1, beta2, eps, step: float, grad_scale: Optional[torch.Tensor] = None):
    """One launch over flat fp32 buffers; ``p16`` (bf16, may be None) receives the rounded parameters."""
    n = p.numel()
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    with torch.cuda.device(p.device):
        rc = lib().ntb_adamw_flat(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _ptr(p16), n, seg_end.data_ptr(), seg_lr.data_ptr(), seg_wd.data_ptr(), seg_end.numel(), beta1, beta2, eps, bc1, bc2, _ptr(grad_scale), _stream(p))
    _check(rc, "adamw_flat")


def multi_tensor_adamw(ps, gs, ms, vs, halves, lr, beta1, beta2, eps, weight_decay, step):
    """Per-tensor launches of the flat kernel (used when the tensors are not one contiguous range)."""
    dev = ps[0].device
    for p, g, m, v, h in zip(ps, gs, ms, vs, halves):
        n = p.numel()
        pad_ok = n % 4 == 0 and all(t.data_ptr() % 16 == 0 for t in (p, g, m, v)) and (h is None or (h.dtype == torch.bfloat16 and h.data_ptr() % 8 == 0))
        if not pad_ok or not g.is_contiguous() or g.dtype != torch.float32:
            from nanotron_b200.ops import reference as ref

            ref.adamw_step(p, g.float(), m, v, lr, beta1, beta2, eps, weight_decay, step)
            if h is not None:
                h.copy_(p.view(-1))
            continue
        seg_end = torch.tensor([n], dtype=torch.int64, device=dev)
        seg_lr = torch.tensor([lr], dtype=torch.float32, device=dev)
        seg_wd = torch.tensor([weight_decay], dtype=torch.float32, device=dev)
        adamw_flat(p.view(-1), g.view(-1), m.view(-1), v.view(-1), h, seg_end, seg_lr, seg_wd, beta1, beta2, eps, step)


def sumsq(x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    L = lib()
    partial = torch.empty(L.ntb_sumsq_num_partials(), dtype=torch.float32, device=x.device)
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = L.ntb_sumsq(x.data_ptr(), x.numel(), partial.data_ptr(), out.data_ptr(), int(accumulate), _stream(x))
    _check(rc, "sumsq")
    return out


# ---------------------------------------------------------------------------- embedding
def embedding_fwd(ids: torch.Tensor, weight: torch.Tensor, min_id: int, max_id: int) -> torch.Tensor:
    """out[..., h] = weight[ids - min_id] for ids in [min_id, max_id), zeros elsewhere."""
    L = lib()
    L.ntb_embedding_fwd.restype = c_int
    L.ntb_embedding_fwd.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p]
    flat = ids.reshape(-1).contiguous()
    out = torch.empty((*ids.shape, weight.shape[1]), dtype=weight.dtype, device=weight.device)
    with torch.cuda.device(weight.device):
        rc = L.ntb_embedding_fwd(_DT[weight.dtype], flat.data_ptr(), weight.data_ptr(), out.data_ptr(), flat.numel(), weight.shape[1], min_id, max_id, _stream(weight))
    _check(rc, "embedding_fwd")
    return out


def embedding_bwd_accum(ids: torch.Tensor, dout: torch.Tensor, dweight_fp32: torch.Tensor, min_id: int, max_id: int) -> None:
    """dweight_fp32[ids - min_id] += dout (fp32 vector atomics)."""
    L = lib()
    L.ntb_embedding_bwd.restype = c_int
    L.ntb_embedding_bwd.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p]
    flat = ids.reshape(-1).contiguous()
    d2 = dout.reshape(-1, dout.shape[-1]).contiguous()
    assert dweight_fp32.dtype == torch.float32 and dweight_fp32.is_contiguous()
    with torch.cuda.device(dout.device):
        rc = L.ntb_embedding_bwd(_DT[d2.dtype], flat.data_ptr(), d2.data_ptr(), dweight_fp32.data_ptr(), flat.numel(), d2.shape[1], min_id, max_id, _stream(dout))
    _check(rc, "embedding_bwd")


# ---------------------------------------------------------------------------- MoE router
def moe_router_supported(x: torch.Tensor, weight: torch.Tensor, k: int) -> bool:
    E = weight.shape[0]
    return x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.float32 and x.is_contiguous() and weight.is_contiguous() and E % 16 == 0 and E <= 128 and x.shape[1] % 8 == 0 and hasattr(lib(), "ntb_moe_router_fwd")


def moe_router_fwd(x: torch.Tensor, weight: torch.Tensor, k: int):
    """Returns (top_p [T,k] fp32, top_i [T,k] int32, probs [T,E] fp32, counts [E] int32)."""
    T, h = x.shape
    E = weight.shape[0]
    L = lib()
    L.ntb_moe_router_fwd.restype = c_int
    L.ntb_moe_router_fwd.argtypes = [c_void_p] * 6 + [c_int] * 4 + [c_void_p]
    probs = torch.empty((T, E), dtype=torch.float32, device=x.device)
    top_p = torch.empty((T, k), dtype=torch.float32, device=x.device)
    top_i = torch.empty((T, k), dtype=torch.int32, device=x.device)
    counts = torch.zeros(E, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        rc = L.ntb_moe_router_fwd(x.data_ptr(), weight.data_ptr(), probs.data_ptr(), top_p.data_ptr(), top_i.data_ptr(), counts.data_ptr(), T, h, E, k, _stream(x))
    _check(rc, "moe_router_fwd")
    return top_p, top_i, probs, counts


# ---------------------------------------------------------------------------- fp8
def has_fp8_quantize() -> bool:
    return hasattr(lib(), "ntb_fp8_quantize_1x128")


def fp8_quantize_1x128(x: torch.Tensor, dtype: torch.dtype):
    from nanotron_b200.fp8.quantize import FP8BlockTensor

    rows, cols = x.shape
    L = lib()
    L.ntb_fp8_quantize_1x128.restype = c_int
    L.ntb_fp8_quantize_1x128.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
    q = torch.empty((rows, cols), dtype=dtype, device=x.device)
    scale = torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = L.ntb_fp8_quantize_1x128(x.data_ptr(), q.data_ptr(), scale.data_ptr(), rows, cols, int(dtype == torch.float8_e5m2), _stream(x))
    _check(rc, "fp8_quantize_1x128")
    return FP8BlockTensor(q, scale, (1, 128))


def has_fp8_gemm() -> bool:
    return hasattr(lib(), "ntb_gemm_fp8_blockscaled")


def gemm_fp8_blockscaled(a, b, out: Optional[torch.Tensor] = None, accumulate_fp32: bool = False, epi_warps: int = 0) -> torch.Tensor:
    """``a`` [M, K] (1 x 128 scales) times ``b`` [N, K]^T (128 x 128 or 1 x 128 scales) on the fp8 tensor cores, with the per-block
    scales applied in fp32 between k-blocks.  Returns bf16 [M, N], or accumulates into the fp32 ``out`` when ``accumulate_fp32``."""
    from nanotron_b200.ops import native_gemm

    M, K = a.data.shape
    N, Kb = b.data.shape
    assert K == Kb and a.block == (1, 128) and b.block in ((1, 128), (128, 128)) and a.data.is_contiguous() and b.data.is_contiguous()
    assert a.scale.is_contiguous() and b.scale.is_contiguous() and a.scale.shape[1] == (K + 127) // 128 == b.scale.shape[1]
    L = lib()
    L.ntb_gemm_fp8_blockscaled.restype = c_int
    L.ntb_gemm_fp8_blockscaled.argtypes = [c_void_p] * 5 + [c_int] * 3 + [c_int64] * 3 + [c_int] * 5 + [c_void_p, c_int, c_void_p]
    if accumulate_fp32:
        assert out is not None and out.dtype == torch.float32 and out.shape == (M, N) and out.is_contiguous()
        mode = 2
    else:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.data.device) if out is None else out
        mode = 0
    status = native_gemm.status_word(a.data.device)
    with torch.cuda.device(a.data.device):
        rc = L.ntb_gemm_fp8_blockscaled(a.data.data_ptr(), a.scale.data_ptr(), b.data.data_ptr(), b.scale.data_ptr(), out.data_ptr(), M, N, K, K, K, N,
                                        int(a.data.dtype == torch.float8_e5m2), int(b.data.dtype == torch.float8_e5m2), int(b.block == (1, 128)), mode, epi_warps,
                                        status.data_ptr(), 0, _stream(a.data))
    _check(rc, "gemm_fp8_blockscaled")
    return out


# ---------------------------------------------------------------------------- GEMM / attention: see native_gemm / native_attn
from nanotron_b200.ops.native_attn import flash_attn_bwd, flash_attn_fwd, flash_attn_supported  # noqa: E402,F401
from nanotron_b200.ops.native_gemm import gemm_nn, gemm_nt, gemm_supported, gemm_tn, gemm_tn_accum_fp32  # noqa: E402,F401
