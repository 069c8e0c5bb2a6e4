"""Linear layer trained with block-scaled fp8 operands (scope parity: reference src/nanotron/fp8/linear.py, whose backward is
a placeholder that replaces grad_output by ones).

Numerics: forward y = dq(q_e4m3^{1x128}(x)) @ dq(q_e4m3^{128x128}(W))^T; backward uses e5m2 1x128 for grad_output in both
dgrad and wgrad, with x and grad_output re-quantised along the token dimension for wgrad.  On CUDA the three products run on the
fp8 tensor cores (``ops/csrc/gemm_fp8.cu``: tcgen05 kind::f8f6f4, per-k-block partial products promoted with the two scales in
fp32); everything is K-major for the kernel, so the weight is also quantised transposed for dgrad (128 x 128 blocks make that a
transpose of payload and scales).  Elsewhere the same numerics are produced by a bf16 / fp32 GEMM over the dequantised operands.
"""
from __future__ import annotations

import torch
from torch import nn

from nanotron_b200 import ops
from nanotron_b200.fp8.parameter import weight_cache
from nanotron_b200.fp8.quantize import dequantize, quantize_1x128


def _native_fp8(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    if not (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and ops.get_mode() != "torch"):
        return False
    from nanotron_b200.ops import native

    M, K = x2.shape
    N = weight.shape[0]
    return native.has_fp8_gemm() and K % 128 == 0 and N % 128 == 0 and M % 128 == 0


def shapes_ok(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    """Block scaling needs every dimension of the product to be a multiple of the 128-element block."""
    return x2.dim() == 2 and weight.dim() == 2 and x2.shape[0] % 128 == 0 and x2.shape[1] % 128 == 0 and weight.shape[0] % 128 == 0 and x2.shape[1] == weight.shape[1]


def fp8_forward(x2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = dq(q_e4m3^{1x128}(x)) @ dq(q_e4m3^{128x128}(W))^T."""
    xq = quantize_1x128(x2, torch.float8_e4m3fn)
    wq = weight_cache.get(weight, torch.float8_e4m3fn)  # quantised once per optimizer step, not once per micro-batch
    if _native_fp8(x2, weight):
        from nanotron_b200.ops import native

        return native.gemm_fp8_blockscaled(xq, wq)
    return torch.nn.functional.linear(dequantize(xq, x2.dtype), dequantize(wq, weight.dtype))


def fp8_dgrad(go: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """dx = dq(q_e5m2^{1x128}(dy)) @ dq(q_e4m3^{128x128}(W))."""
    go = go.contiguous()
    if go.is_cuda and go.dtype == torch.bfloat16 and _native_fp8(go, weight.t()):
        from nanotron_b200.ops import native

        goq = quantize_1x128(go, torch.float8_e5m2)
        wq_t = weight_cache.get(weight, torch.float8_e4m3fn, transposed=True)  # [K, N]: K-major for the dgrad reduction over N
        return native.gemm_fp8_blockscaled(goq, wq_t)
    goq = dequantize(quantize_1x128(go, torch.float8_e5m2), go.dtype)
    wq = dequantize(weight_cache.get(weight, torch.float8_e4m3fn), weight.dtype)
    return goq.matmul(wq)


def fp8_wgrad(go: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor):
    """dW = dy^T x with both operands quantised in 1 x 128 blocks along the token dimension (the reduction dimension of this
    product).  Accumulates into ``weight.main_grad`` (fp32) when there is one and then returns None."""
    go = go.contiguous()
    main_grad = getattr(weight, "main_grad", None)
    if go.is_cuda and go.dtype == torch.bfloat16 and _native_fp8(x2, weight):
        from nanotron_b200.ops import native

        go_t = quantize_1x128(go.t().contiguous(), torch.float8_e5m2)  # [N, M], blocks along the tokens
        x_t = quantize_1x128(x2.t().contiguous(), torch.float8_e4m3fn)  # [K, M]
        if main_grad is not None:
            native.gemm_fp8_blockscaled(go_t, x_t, out=main_grad, accumulate_fp32=True)
            return None
        return native.gemm_fp8_blockscaled(go_t, x_t)
    go_t = dequantize(quantize_1x128(go.t().contiguous(), torch.float8_e5m2), go.dtype)
    x_t = dequantize(quantize_1x128(x2.t().contiguous(), torch.float8_e4m3fn), x2.dtype)
    dw = go_t.matmul(x_t.t())
    if main_grad is not None:
        main_grad.add_(dw)
        return None
    return dw


class _FP8Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weight):
        ctx.save_for_backward(x2, weight)
        return fp8_forward(x2, weight)

    @staticmethod
    def backward(ctx, grad_out):
        x2, weight = ctx.saved_tensors
        return fp8_dgrad(grad_out, weight), fp8_wgrad(grad_out, x2, weight)


class FP8Linear(nn.Linear):
    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x2 = input.reshape(-1, input.shape[-1])
        y = _FP8Matmul.apply(x2, self.weight)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*input.shape[:-1], self.out_features)
