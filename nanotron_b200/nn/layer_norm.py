"""Normalisation layers.  ``TritonRMSNorm`` / ``TritonLayerNorm`` keep the reference's class names
(reference src/nanotron/nn/layer_norm.py:6-75) but run the in-tree sm_100a kernels (fp32 statistics, optional fused
residual add) on CUDA and the PyTorch oracle on CPU."""
from __future__ import annotations

import torch
from torch import nn

from nanotron_b200 import ops


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.empty(hidden_size, device=device, dtype=dtype))
        self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, input, residual=None, dropout_p=0.0, prenorm=False, residual_in_fp32=False, return_dropout_mask=False):
        """With ``residual``: returns (norm(input + residual), input + residual).  With ``prenorm`` and no residual: returns
        (norm(input), input); taking the skip connection from that second output lets the backward kernel sum the two
        gradient paths of ``input`` itself."""
        assert dropout_p == 0.0 and not return_dropout_mask, "dropout inside the norm is not supported"
        return ops.rms_norm(input, self.weight, self.eps, residual=residual, return_input=prenorm and residual is None)


class LayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5, bias=True, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.empty(normalized_shape, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(normalized_shape, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.ones_(self.weight)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, input, residual=None, dropout_p=0.0, prenorm=False, residual_in_fp32=False, return_dropout_mask=False):
        assert dropout_p == 0.0 and not return_dropout_mask
        return ops.layer_norm(input, self.weight, self.bias, self.eps, residual=residual)


TritonRMSNorm = RMSNorm
TritonLayerNorm = LayerNorm


class LlamaRMSNorm(nn.Module):
    """Eager fp32 RMSNorm, always the PyTorch math (the oracle the fused kernel is tested against)."""

    def __init__(self, hidden_size, eps=1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.variance_epsilon = eps

    def forward(self, input):
        dtype = input.dtype
        x = input.to(torch.float32)
        variance = x.pow(2).mean(-1, keepdim=True)
        x = x * torch.rsqrt(variance + self.variance_epsilon)
        return (self.weight.float() * x).to(dtype)
