"""Bindings of the flash-attention kernels (``csrc/attention_fwd2.cu``: two query tiles per CTA, the default forward;
``csrc/attention_fwd.cu``: one query tile per CTA, also the context-parallel forward; ``csrc/attention_bwd.cu``)."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

_HAS = {"fwd": False, "fwd2": False, "bwd": False}
FWD_VARIANT = {"kernel": "two_tile"}  # "two_tile" | "one_tile"
BWD_SPLIT = {"mode": "auto"}  # "auto" (by launch size) | "on" | "off": one backward CTA per query head instead of per kv head


def set_forward_variant(name: str):
    assert name in ("two_tile", "one_tile")
    FWD_VARIANT["kernel"] = name


def declare(L):
    _HAS["fwd"] = hasattr(L, "ntb_flash_attn_fwd")
    _HAS["bwd"] = hasattr(L, "ntb_flash_attn_bwd")
    if _HAS["fwd"]:
        L.ntb_flash_attn_fwd.restype = c_int
        L.ntb_flash_attn_fwd.argtypes = [c_void_p] * 7 + [c_int] * 6 + [c_int64] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p]
    _HAS["fwd2"] = hasattr(L, "ntb_flash_attn_fwd2")
    if _HAS["fwd2"]:
        L.ntb_flash_attn_fwd2.restype = c_int
        L.ntb_flash_attn_fwd2.argtypes = L.ntb_flash_attn_fwd.argtypes
    if _HAS["bwd"]:
        L.ntb_flash_attn_bwd.restype = c_int
        L.ntb_flash_attn_bwd.argtypes = [c_void_p] * 13 + [c_int] * 7 + [c_int64] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p]
        L.ntb_flash_attn_bwd_split.restype = c_int
        L.ntb_flash_attn_bwd_split.argtypes = [c_void_p] * 14 + [c_int] * 7 + [c_int64] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p]
        L.ntb_flash_attn_bwd_wants_split.restype = c_int
        L.ntb_flash_attn_bwd_wants_split.argtypes = [c_int] * 4


def _ok(t: torch.Tensor) -> bool:
    return t.dim() == 3 and t.dtype == torch.bfloat16 and t.shape[-1] == 128 and t.stride(-1) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0


def flash_attn_supported(q, k, v, window, need_backward: bool = True) -> bool:
    """Head dim 128, bf16, last dim contiguous.  Training also needs the backward kernel."""
    from nanotron_b200.ops import native

    native.lib()
    if not _HAS["fwd"] or (need_backward and not _HAS["bwd"]):
        return False
    return _ok(q) and _ok(k) and _ok(v) and q.shape[1] % k.shape[1] == 0


def flash_attn_fwd(q, k, v, cu_q, cu_k, max_q: int, max_k: int, causal: bool, scale: float, window: Optional[int]):
    from nanotron_b200.ops import native
    from nanotron_b200.ops.native_gemm import status_word

    Tq, Hq, D = q.shape
    out = torch.empty((Tq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device)
    cu_q = cu_q.to(torch.int32)
    cu_k = cu_k.to(torch.int32)
    L = native.lib()
    fn = L.ntb_flash_attn_fwd2 if (_HAS["fwd2"] and FWD_VARIANT["kernel"] == "two_tile") else L.ntb_flash_attn_fwd
    with torch.cuda.device(q.device):
        rc = fn(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), cu_q.data_ptr(), cu_k.data_ptr(), cu_q.numel() - 1, int(max_q), Tq, k.shape[0],
            Hq, k.shape[1], q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), float(scale), int(bool(causal)), int(window or 0),
            status_word(q.device).data_ptr(), torch.cuda.current_stream(q.device).cuda_stream,
        )
    native._check(rc, "flash_attn_fwd")
    return out, lse


def flash_attn_bwd(dout, q, k, v, out, lse, cu_q, cu_k, max_q: int, max_k: int, causal: bool, scale: float, window: Optional[int]):
    from nanotron_b200.ops import native
    from nanotron_b200.ops.native_gemm import status_word

    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    # one fused buffer so the gradient of a fused qkv projection needs no concatenation
    dqkv = torch.empty((Tq, Hq + 2 * Hkv, D), dtype=q.dtype, device=q.device) if Tq == Tk else None
    if dqkv is not None:
        dq, dk, dv = dqkv[:, :Hq], dqkv[:, Hq : Hq + Hkv], dqkv[:, Hq + Hkv :]
    else:
        dq, dk, dv = torch.empty_like(q), torch.empty((Tk, Hkv, D), dtype=k.dtype, device=k.device), torch.empty((Tk, Hkv, D), dtype=v.dtype, device=v.device)
    dq_acc = torch.zeros((Tq, Hq, D), dtype=torch.float32, device=q.device)
    delta = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device)
    cu_q = cu_q.to(torch.int32)
    cu_k = cu_k.to(torch.int32)
    L = native.lib()
    batch = cu_q.numel() - 1
    split = BWD_SPLIT["mode"] == "on" or (BWD_SPLIT["mode"] == "auto" and L.ntb_flash_attn_bwd_wants_split(batch, int(max_k), Hq, Hkv) == 1)
    tail = (
        cu_q.data_ptr(), cu_k.data_ptr(), batch, int(max_q), int(max_k), Tq, Tk, Hq, Hkv,
        q.stride(0), q.stride(1), k.stride(0), k.stride(1), dq.stride(0), dk.stride(0), float(scale), int(bool(causal)), int(window or 0),
        status_word(q.device).data_ptr(), torch.cuda.current_stream(q.device).cuda_stream,
    )
    head = (dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr())
    with torch.cuda.device(q.device):
        if split and Hq != Hkv:
            # too few (key tile, kv head) pairs to fill the GPU: one CTA per query head, dK / dV summed in fp32 scratch
            dkv_acc = torch.zeros((2, Tk, Hkv, D), dtype=torch.float32, device=q.device)
            rc = L.ntb_flash_attn_bwd_split(*head, dkv_acc.data_ptr(), *tail)
        else:
            rc = L.ntb_flash_attn_bwd(*head, *tail)
    native._check(rc, "flash_attn_bwd")
    return dq, dk, dv
