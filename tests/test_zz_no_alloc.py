"""The allocation-free RMSNorm backward, called through its exported C symbol.

Who needs it: code that runs while device memory is frozen (runtimes that reserve all memory up front, hooks inside
another allocator) cannot hand the kernel a freshly allocated scratch buffer.
The variant keeps its scratch inside the library image; here it must reproduce the regular entry point, twice in a row
(the second call reuses the same scratch), and refuse rows wider than its built-in limit.
This file sorts last on purpose: a failure here cannot hide failures of the other GPU tests in a stop-at-first-failure run.
"""
import ctypes
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


@pytest.mark.parametrize("rows,cols,dtype", [(333, 4096, torch.bfloat16), (64, 1024, torch.float32)])
def test_noalloc_rmsnorm_bwd_matches_regular_entry_point(rows, cols, dtype):
    from nanotron_b200.ops import native

    L = _lib()
    code = {torch.float32: 0, torch.bfloat16: 1}[dtype]
    stream = torch.cuda.current_stream().cuda_stream
    for trial in range(2):  # two calls in a row share the built-in scratch
        torch.manual_seed(trial)
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        res = torch.randn(rows, cols, device="cuda", dtype=dtype)
        w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype)
        _, pre, rstd = native.rmsnorm_fwd(x, res, w, 1e-5)
        dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dres = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dx_ref, dw_ref = native.rmsnorm_bwd(dy, pre, w, rstd, dres)
        dx = torch.empty_like(dx_ref)
        dw = torch.empty(cols, device="cuda", dtype=torch.float32)
        rc = L.ntb_rmsnorm_bwd_noalloc(code, dy.data_ptr(), pre.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, cols, stream)
        assert rc == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5)
        # the two entry points split rows over a different number of CTAs, so dW differs by fp32 summation order only
        torch.testing.assert_close(dw, dw_ref, atol=5e-2 if dtype == torch.bfloat16 else 1e-3, rtol=2e-2)


def test_noalloc_rejects_rows_wider_than_its_scratch():
    L = _lib()
    limit = L.ntb_rmsnorm_bwd_noalloc_max_cols()
    assert limit == 8192
    rc = L.ntb_rmsnorm_bwd_noalloc(1, None, None, None, None, None, None, None, 4, limit + 8, None)
    assert rc == 1
