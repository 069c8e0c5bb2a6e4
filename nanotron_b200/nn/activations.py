"""Activation registry keyed by the names used in model configs (parity: reference src/nanotron/nn/activations.py)."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch
from torch import nn


class NewGELUActivation(nn.Module):
    def forward(self, x):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * torch.pow(x, 3.0))))


class PytorchGELUTanh(nn.Module):
    def forward(self, x):
        return nn.functional.gelu(x, approximate="tanh")


class FastGELUActivation(nn.Module):
    def forward(self, x):
        return 0.5 * x * (1.0 + torch.tanh(x * 0.7978845608 * (1.0 + 0.044715 * x * x)))


class QuickGELUActivation(nn.Module):
    def forward(self, x):
        return x * torch.sigmoid(1.702 * x)


class ClippedGELUActivation(nn.Module):
    def __init__(self, min: float, max: float):
        if min > max:
            raise ValueError(f"min should be < max (got min: {min}, max: {max})")
        super().__init__()
        self.min, self.max = min, max

    def forward(self, x):
        return torch.clip(nn.functional.gelu(x), self.min, self.max)


class AccurateGELUActivation(nn.Module):
    def __init__(self):
        super().__init__()
        self.precomputed_constant = math.sqrt(2 / math.pi)

    def forward(self, x):
        return 0.5 * x * (1 + torch.tanh(self.precomputed_constant * (x + 0.044715 * torch.pow(x, 3))))


class LaplaceActivation(nn.Module):
    def forward(self, x, mu=0.707107, sigma=0.282095):
        return 0.5 * (1.0 + torch.erf((x - mu) / (sigma * math.sqrt(2.0))))


class ReLUSquaredActivation(nn.Module):
    def forward(self, x):
        return torch.square(nn.functional.relu(x))


class LinearActivation(nn.Module):
    def forward(self, x):
        return x


class ClassInstantier(OrderedDict):
    def __getitem__(self, key):
        content = super().__getitem__(key)
        cls, kwargs = content if isinstance(content, tuple) else (content, {})
        return cls(**kwargs)


ACT2CLS = {
    "gelu": nn.GELU,
    "gelu_10": (ClippedGELUActivation, {"min": -10, "max": 10}),
    "gelu_fast": FastGELUActivation,
    "gelu_new": NewGELUActivation,
    "gelu_python": nn.GELU,
    "gelu_pytorch_tanh": PytorchGELUTanh,
    "gelu_accurate": AccurateGELUActivation,
    "laplace": LaplaceActivation,
    "linear": LinearActivation,
    "mish": nn.Mish,
    "quick_gelu": QuickGELUActivation,
    "relu": nn.ReLU,
    "relu2": ReLUSquaredActivation,
    "relu6": nn.ReLU6,
    "sigmoid": nn.Sigmoid,
    "silu": nn.SiLU,
    "swish": nn.SiLU,
    "tanh": nn.Tanh,
}
ACT2FN = ClassInstantier(ACT2CLS)


def get_activation(name: str):
    if name in ACT2FN:
        return ACT2FN[name]
    raise KeyError(f"function {name} not found in ACT2FN mapping {list(ACT2FN.keys())}")


class GLUActivation(nn.Module):
    """act(gate) * up over a fused [gate | up] tensor; "silu" uses the fused SwiGLU kernel."""

    def __init__(self, act_fn_name: str):
        super().__init__()
        self.name = act_fn_name
        self.act = ACT2FN[act_fn_name]

    def forward(self, merged_states: torch.Tensor):
        if self.name in ("silu", "swish"):
            from nanotron_b200 import ops

            return ops.swiglu(merged_states)
        gate, up = torch.split(merged_states, merged_states.shape[-1] // 2, dim=-1)
        return self.act(gate) * up
