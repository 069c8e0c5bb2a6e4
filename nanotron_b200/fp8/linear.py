"""Linear layer trained with block-scaled fp8 operands (scope parity: reference src/nanotron/fp8/linear.py, whose backward is
a placeholder that replaces grad_output by ones).

Numerics implemented here: forward y = dq(q_e4m3^{1x128}(x)) @ dq(q_e4m3^{128x128}(W))^T; backward uses e5m2 1x128 for
grad_output in both dgrad and wgrad, with x re-quantised along the token dimension for wgrad.  The products currently run on
the bf16 tensor-core GEMM over the dequantised operands (so the result has exactly the block-scaled fp8 rounding of the
operands, accumulated in fp32); a kind::f8f6f4 tcgen05 kernel consuming the payloads and scales directly is the intended
replacement and would not change these numerics.
"""
from __future__ import annotations

import torch
from torch import nn

from nanotron_b200 import ops
from nanotron_b200.fp8.quantize import dequantize, quantize_1x128, quantize_128x128


class _FP8Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weight):
        xq = quantize_1x128(x2, torch.float8_e4m3fn)
        wq = quantize_128x128(weight, torch.float8_e4m3fn)
        ctx.save_for_backward(x2, weight)
        return ops.linear_forward(dequantize(xq, x2.dtype), dequantize(wq, weight.dtype))

    @staticmethod
    def backward(ctx, grad_out):
        x2, weight = ctx.saved_tensors
        go = grad_out.contiguous()
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
