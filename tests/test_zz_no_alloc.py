"""The allocation-free RMSNorm backward, called through its exported C symbol.

Who needs it: code that runs while device memory is frozen (runtimes that reserve all memory up front, hooks inside
another allocator) cannot hand the kernel a freshly allocated scratch buffer.
The variant keeps its scratch inside the library image; here it must reproduce the regular entry point, twice in a row
(the second call reuses the same scratch), and refuse rows wider than its built-in limit.
This file sorts last on purpose: a failure here cannot hide failures of the other GPU tests in a stop-at-first-failure run.
"""
import ctypes
import gc
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from nanotron_b200.ops import native

    L = native.lib()
    L.ntb_rmsnorm_bwd_noalloc.restype = c_int
    L.ntb_rmsnorm_bwd_noalloc.argtypes = [c_int] + [c_void_p] * 7 + [c_int, c_int, c_void_p]
    L.ntb_rmsnorm_bwd_noalloc_max_cols.restype = c_int
    return L


def _oracle(dy, pre, w, dres, eps=1e-5):
    """RMSNorm backward in plain fp32 PyTorch: y = pre * rsqrt(mean(pre^2) + eps) * w, dres added to the input gradient."""
    pre32 = pre.float().detach().requires_grad_(True)
    w32 = w.float().detach().requires_grad_(True)
    y = pre32 * torch.rsqrt(pre32.pow(2).mean(-1, keepdim=True) + eps) * w32
    y.backward(dy.float())
    dx = pre32.grad if dres is None else pre32.grad + dres.float()
    return dx, w32.grad


@pytest.mark.parametrize(
    "rows,cols,dtype,with_dres",
    [(333, 4096, torch.bfloat16, True), (64, 1024, torch.float32, True), (200, 8192, torch.bfloat16, True), (40, 2048, torch.float32, False)],
)
def test_noalloc_rmsnorm_bwd_matches_regular_entry_point(rows, cols, dtype, with_dres):
    from nanotron_b200.ops import native

    L = _lib()
    code = {torch.float32: 0, torch.bfloat16: 1}[dtype]
    stream = torch.cuda.current_stream().cuda_stream
    half = dtype == torch.bfloat16
    for trial in range(2):  # two calls in a row share the built-in scratch
        torch.manual_seed(trial)
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        res = torch.randn(rows, cols, device="cuda", dtype=dtype)
        w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype)
        y, pre, rstd = native.rmsnorm_fwd(x, res, w, 1e-5)
        del y
        dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dres = torch.randn(rows, cols, device="cuda", dtype=dtype) if with_dres else None
        dx_ref, dw_ref = native.rmsnorm_bwd(dy, pre, w, rstd, dres)
        dx = torch.empty_like(dx_ref)
        dw = torch.empty(cols, device="cuda", dtype=torch.float32)
        gc.collect()  # nothing of earlier work may be released inside the measured window
        torch.cuda.synchronize()
        # the call must leave the device's memory accounting untouched: nothing allocated through torch, nothing through the CUDA
        # runtime (the second trial also covers the first call's one-time symbol look-up having been paid already)
        torch_before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = L.ntb_rmsnorm_bwd_noalloc(code, dy.data_ptr(), pre.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if with_dres else None, dx.data_ptr(), dw.data_ptr(), rows, cols, stream)
        torch.cuda.synchronize()
        torch_after, free_after = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert rc == 0
        assert torch_after == torch_before, (torch_before, torch_after)
        dx_or, dw_or = _oracle(dy, pre, w, dres)
        if trial == 1:
            assert free_after == free_before, (free_before, free_after)
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=2e-2 if half else 1e-5, rtol=2e-2 if half else 1e-5)
        # the two entry points split rows over a different number of CTAs, so dW differs by fp32 summation order only
        torch.testing.assert_close(dw, dw_ref, atol=5e-2 if half else 1e-3, rtol=2e-2)
        # and against the fp32 PyTorch formula (bf16 inputs: dx is rounded to bf16 on the way out)
        torch.testing.assert_close(dx.float(), dx_or, atol=6e-2 if half else 1e-4, rtol=2e-2 if half else 1e-4)
        torch.testing.assert_close(dw, dw_or, atol=2e-1 if half else 1e-3, rtol=2e-2)


def test_noalloc_rejects_rows_wider_than_its_scratch():
    L = _lib()
    limit = L.ntb_rmsnorm_bwd_noalloc_max_cols()
    assert limit == 8192
    rc = L.ntb_rmsnorm_bwd_noalloc(1, None, None, None, None, None, None, None, 4, limit + 8, None)
    assert rc == 1
