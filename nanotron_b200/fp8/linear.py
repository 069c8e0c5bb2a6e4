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
from nanotron_b200.fp8.quantize import dequantize, quantize_1x128, quantize_128x128


def _native_fp8(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    if not (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and ops.get_mode() != "torch"):
        return False
    from nanotron_b200.ops import native

    M, K = x2.shape
    N = weight.shape[0]
    return native.has_fp8_gemm() and K % 128 == 0 and N % 128 == 0 and M % 128 == 0


def _transpose_blocks(t):
    """Transposed view of a 128 x 128-block tensor as a new block tensor (payload and scales transposed)."""
    from nanotron_b200.fp8.quantize import FP8BlockTensor

    return FP8BlockTensor(t.data.t().contiguous(), t.scale.t().contiguous(), t.block)


class _FP8Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weight):
        xq = quantize_1x128(x2, torch.float8_e4m3fn)
        wq = quantize_128x128(weight, torch.float8_e4m3fn)
        ctx.save_for_backward(x2, weight)
        if _native_fp8(x2, weight):
            from nanotron_b200.ops import native

            return native.gemm_fp8_blockscaled(xq, wq)
        return ops.linear_forward(dequantize(xq, x2.dtype), dequantize(wq, weight.dtype))

    @staticmethod
    def backward(ctx, grad_out):
        x2, weight = ctx.saved_tensors
        go = grad_out.contiguous()
        if _native_fp8(x2, weight) and go.dtype == torch.bfloat16:
            from nanotron_b200.ops import native

            goq = quantize_1x128(go, torch.float8_e5m2)
            wq_t = _transpose_blocks(quantize_128x128(weight, torch.float8_e4m3fn))  # [K, N]: K-major for the dgrad reduction over N
            dx = native.gemm_fp8_blockscaled(goq, wq_t)
            go_t = quantize_1x128(go.t().contiguous(), torch.float8_e5m2)  # [N, M], blocks along the tokens
            x_t = quantize_1x128(x2.t().contiguous(), torch.float8_e4m3fn)  # [K, M]
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                native.gemm_fp8_blockscaled(go_t, x_t, out=main_grad, accumulate_fp32=True)
                return dx, None
            return dx, native.gemm_fp8_blockscaled(go_t, x_t)
        goq = dequantize(quantize_1x128(go, torch.float8_e5m2), go.dtype)
        wq = dequantize(quantize_128x128(weight, torch.float8_e4m3fn), weight.dtype)
        dx = ops.linear_dgrad(goq, wq)
        # wgrad contracts over tokens: quantise both operands in blocks along that dimension (transposed 1x128)
        go_t = dequantize(quantize_1x128(go.t().contiguous(), torch.float8_e5m2), go.dtype).t()
        x_t = dequantize(quantize_1x128(x2.t().contiguous(), torch.float8_e4m3fn), x2.dtype).t()
        dw = ops.linear_wgrad(go_t.contiguous(), x_t.contiguous(), weight)
        return dx, dw


class FP8Linear(nn.Linear):
    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x2 = input.reshape(-1, input.shape[-1])
        y = _FP8Matmul.apply(x2, self.weight)
        if self.bias is not None:
            y = y + self.bias
        return y.view(*input.shape[:-1], self.out_features)
