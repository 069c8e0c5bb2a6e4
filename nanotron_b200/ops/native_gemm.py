"""Bindings of the tcgen05 GEMM kernel (``csrc/gemm_tcgen05.cu``).

Three products of a linear layer, none of which needs a transposed copy:
  gemm_nt : y[M,N]  = x[M,K] @ w[N,K]^T        (forward)
  gemm_nn : dx[M,K] = dy[M,N] @ w[N,K]          (dgrad; w is read as an MN-major operand)
  gemm_tn : dw[N,K] = dy[M,N]^T @ x[M,K]        (wgrad; both operands MN-major), optionally accumulated in fp32
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_void_p
from typing import Optional

import torch

_HAS = {"gemm": False, "pair": False}
# "single": one CTA per 128 x 256 tile (gemm_tcgen05.cu); "pair": two CTAs per 256 x 256 tile with cta_group::2 (gemm2_tcgen05.cu)
VARIANT = {"kernel": "pair"}


def set_variant(name: str):
    assert name in ("single", "pair")
    VARIANT["kernel"] = name
_STATUS = {}
_SMS = {}
_WORKSPACE = {}  # device -> (fp32 tensor, stream handle) registered with the pair kernel
SPLIT_SLABS = 74  # one workspace slab per CTA pair is the most a launch can use


def ensure_workspace(device) -> None:
    """The pair kernel cuts the tiles of a launch's last, partly filled round along K so that every CTA pair shares the tail;
    each chunk parks its fp32 partial sums in a slab of this scratch (19 MB per device) and a fix-up pass sums them in a fixed
    order.  The scratch belongs to the stream that first launched a GEMM on the device; launches on other streams run unsplit."""
    key = str(device)
    if key in _WORKSPACE or not _HAS["pair"]:
        return
    from nanotron_b200.ops import native

    L = native.lib()
    if not hasattr(L, "ntb_gemm2_set_workspace"):
        _WORKSPACE[key] = None
        return
    ws = torch.empty(SPLIT_SLABS * 256 * 256, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    with torch.cuda.device(device):
        native._check(L.ntb_gemm2_set_workspace(ws.data_ptr(), SPLIT_SLABS, stream), "gemm2 workspace")
    _WORKSPACE[key] = (ws, stream)


def set_split(on: bool) -> None:
    """True lets pair-kernel launches cut the tiles of their last round along K (off by default: on Llama-3-8B shapes it measured
    within +-5 % of whole tiles, because a power-capped B200 is bound by total work rather than by rounds of tiles)."""
    from nanotron_b200.ops import native

    L = native.lib()
    if hasattr(L, "ntb_gemm2_enable_split"):
        L.ntb_gemm2_enable_split(1 if on else 0)


def declare(L):
    _HAS["gemm"] = hasattr(L, "ntb_gemm_bf16")
    if _HAS["gemm"]:
        L.ntb_gemm_bf16.restype = c_int
        L.ntb_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
    _HAS["pair"] = hasattr(L, "ntb_gemm2_bf16")
    if _HAS["pair"]:
        L.ntb_gemm2_bf16.restype = c_int
        L.ntb_gemm2_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        if hasattr(L, "ntb_gemm2_set_workspace"):
            L.ntb_gemm2_set_workspace.restype = c_int
            L.ntb_gemm2_set_workspace.argtypes = [c_void_p, c_int, c_void_p]
            L.ntb_gemm2_enable_split.restype = None
            L.ntb_gemm2_enable_split.argtypes = [c_int]


def status_word(device) -> torch.Tensor:
    """Device int that a kernel sets when one of its bounded waits expired (0 = fine)."""
    key = str(device)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device) -> None:
    """Host-side check (synchronises): raises if any tcgen05 kernel reported a timed-out wait since the last check."""
    from nanotron_b200.ops.native import NativeKernelError

    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise NativeKernelError(f"a tensor-core kernel gave up waiting on a barrier (status {v})")


def _sms(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[key]


def _ok2d(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.data_ptr() % 16 == 0 and t.dtype == torch.bfloat16


def gemm_supported(a: torch.Tensor, b: torch.Tensor, force: bool = False) -> bool:
    """The kernel covers bf16 row-major operands with 16-byte aligned rows; tiny problems stay on the library."""
    if not _HAS["gemm"] and not force:
        from nanotron_b200.ops import native

        native.lib()
    if not _HAS["gemm"]:
        return False
    if not (_ok2d(a) and _ok2d(b)):
        return False
    if a.stride(0) % 64 or b.stride(0) % 64 or a.shape[1] % 64 or b.shape[1] % 64 or a.shape[0] % 64 or b.shape[0] % 64:
        return False  # keeps every (nt, nn, tn) use of the same tensors legal
    if not force and a.shape[0] * a.shape[1] < 512 * 512:
        return False
    return True


def _launch(a, b, d, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_mode):
    from nanotron_b200.ops import native

    dev = a.device
    L = native.lib()
    pair = VARIANT["kernel"] == "pair" and _HAS["pair"]
    fn = L.ntb_gemm2_bf16 if pair else L.ntb_gemm_bf16
    if pair:
        ensure_workspace(dev)
    with torch.cuda.device(dev):
        rc = fn(a.data_ptr(), b.data_ptr(), d.data_ptr(), M, N, K, lda, ldb, ldd, a_mn, b_mn, out_mode, status_word(dev).data_ptr(), _sms(dev), torch.cuda.current_stream(dev).cuda_stream)
    if rc != 0:
        reject = L.ntb_gemm2_last_reject() if hasattr(L, "ntb_gemm2_last_reject") else -1
        what = (f"gemm_tcgen05[{VARIANT['kernel']}] check#{reject} M={M} N={N} K={K} lda={lda} ldb={ldb} ldd={ldd} a_mn={a_mn} b_mn={b_mn} out_mode={out_mode} "
                f"a={tuple(a.shape)}/{a.stride()}/{a.dtype}/ptr%16={a.data_ptr() % 16} b={tuple(b.shape)}/{b.stride()}/{b.dtype}/ptr%16={b.data_ptr() % 16} "
                f"d={tuple(d.shape)}/{d.stride()}/{d.dtype}/ptr%16={d.data_ptr() % 16}")
        native._check(rc, what)
    native._check(0, "gemm_tcgen05")  # counts the launch
    return d


def gemm_nt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    d = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=x.device)
    return _launch(x, w, d, M, N, K, x.stride(0), w.stride(0), d.stride(0), 0, 0, 0 if d.dtype == torch.bfloat16 else 1)


def gemm_nn(dy: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    M, N = dy.shape
    K = w.shape[1]
    d = out if out is not None else torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    return _launch(dy, w, d, M, K, N, dy.stride(0), w.stride(0), d.stride(0), 0, 1, 0 if d.dtype == torch.bfloat16 else 1)


def gemm_tn(dy: torch.Tensor, x: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    M, N = dy.shape
    K = x.shape[1]
    d = torch.empty((N, K), dtype=out_dtype, device=dy.device)
    return _launch(dy, x, d, N, K, M, dy.stride(0), x.stride(0), d.stride(0), 1, 1, 0 if out_dtype == torch.bfloat16 else 1)


def gemm_tn_accum_fp32(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[N,K] (fp32) += dy[M,N]^T @ x[M,K]."""
    M, N = dy.shape
    K = x.shape[1]
    assert out.dtype == torch.float32 and out.shape == (N, K) and out.stride(1) == 1
    return _launch(dy, x, out, N, K, M, dy.stride(0), x.stride(0), out.stride(0), 1, 1, 2)
