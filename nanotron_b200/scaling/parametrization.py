"""Weight initialisation and per-parameter learning rates for standard and spectral-muP parametrisations
(parity: reference src/nanotron/scaling/parametrization.py:19-249)."""
from __future__ import annotations

import math
from abc import abstractmethod
from enum import Enum, auto
from typing import Dict

from torch import nn
from torch.nn import init

from nanotron_b200.config.utils_config import InitScalingMethod
from nanotron_b200.parallel.tensor_parallel.nn import (
    TensorParallelColumnLinear,
    TensorParallelEmbedding,
    TensorParallelRowLinear,
)


class ParametrizationMethod(Enum):
    STANDARD = auto()
    SPECTRAL_MUP = auto()


def _norm_types():
    from nanotron_b200.nn.layer_norm import LayerNorm, LlamaRMSNorm, RMSNorm

    return (RMSNorm, LayerNorm, LlamaRMSNorm, nn.LayerNorm)


def _moe_types():
    from nanotron_b200.nn.moe import GroupedMLP, Router

    return Router, GroupedMLP


class Parametrizator:
    def __init__(self, config):
        self.config = config

    def parametrize(self, param_name: str, module: nn.Module):
        for types, fn in self.MODULE_TO_PARAMETRIZE():
            if isinstance(module, types):
                return fn(param_name, module)
        raise Exception(f"Module {type(module)} with parameter {param_name} is not supported for initialization")

    @abstractmethod
    def MODULE_TO_PARAMETRIZE(self):
        ...


class StandardParametrizator(Parametrizator):
    """normal(0, std) everywhere; output projections (row linears, expert down projections) use
    std / sqrt(2 * num_layers) when ``scaling_method`` is NUM_LAYERS; norm weights are ones, biases zeros."""

    def __init__(self, config):
        super().__init__(config)
        self.std = config.model.init_method.std
        self.num_layers = config.model.model_config.num_hidden_layers
        self.scaling_method = getattr(config.model.init_method, "scaling_method", InitScalingMethod.NUM_LAYERS)

    def MODULE_TO_PARAMETRIZE(self):
        router, grouped = _moe_types()
        return [
            (TensorParallelColumnLinear, self._parametrize_column_linear),
            (TensorParallelRowLinear, self._parametrize_row_linear),
            (_norm_types(), self._parametrize_layer_norm),
            (TensorParallelEmbedding, self._parametrize_embedding),
            (router, self._parametrize_column_linear),
            (grouped, self._parametrize_grouped_mlp),
            (nn.Linear, self._parametrize_column_linear),
        ]

    def _scaling(self) -> float:
        if self.scaling_method == InitScalingMethod.NUM_LAYERS:
            return math.sqrt(2 * self.num_layers)
        if self.scaling_method == InitScalingMethod.NONE:
            return 1.0
        raise ValueError(f"Invalid scaling method: {self.scaling_method}")

    def _parametrize_column_linear(self, param_name: str, module: nn.Module):
        p = dict(module.named_parameters(recurse=False))[param_name.rpartition(".")[2]]
        if "weight" in param_name.rpartition(".")[2]:
            init.normal_(p, mean=0.0, std=self.std)
        else:
            p.zero_()

    def _parametrize_row_linear(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        if "weight" in local:
            init.normal_(p, mean=0.0, std=self.std / self._scaling())
        else:
            p.zero_()

    def _parametrize_grouped_mlp(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        if local == "merged_down_proj":
            init.normal_(p, mean=0.0, std=self.std / self._scaling())
        else:
            init.normal_(p, mean=0.0, std=self.std)

    def _parametrize_layer_norm(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        if "weight" in local:
            p.fill_(1)
        else:
            p.zero_()

    def _parametrize_embedding(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        init.normal_(p, mean=0.0, std=self.std)


class SpectralMupParametrizator(Parametrizator):
    """sigma = (1/sqrt(fan_in)) * min(1, sqrt(fan_out/fan_in)) on the *unsharded* fan sizes."""

    def MODULE_TO_PARAMETRIZE(self):
        return [
            (TensorParallelColumnLinear, self._parametrize_mup_weight),
            (TensorParallelRowLinear, self._parametrize_mup_weight),
            (_norm_types(), self._parametrize_layer_norm),
            (TensorParallelEmbedding, self._parametrize_embedding),
        ]

    @staticmethod
    def _compute_spectral_std(std: float, fan_in: int, fan_out: int) -> float:
        return (std / math.sqrt(fan_in)) * min(1, math.sqrt(fan_out / fan_in))

    def _parametrize_mup_weight(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        if "weight" not in local:
            p.zero_()
            return
        fan_in, fan_out = _unsharded_fans(module)
        init.normal_(p, mean=0.0, std=self._compute_spectral_std(1.0, fan_in, fan_out))

    def _parametrize_layer_norm(self, param_name: str, module: nn.Module):
        local = param_name.rpartition(".")[2]
        p = dict(module.named_parameters(recurse=False))[local]
        p.fill_(1) if "weight" in local else p.zero_()

    def _parametrize_embedding(self, param_name: str, module: nn.Module):
        p = dict(module.named_parameters(recurse=False))[param_name.rpartition(".")[2]]
        init.normal_(p, mean=0.0, std=1.0)


def _unsharded_fans(module):
    world = module.world_size
    if isinstance(module, TensorParallelColumnLinear):
        return module.in_features, module.out_features * world
    if isinstance(module, TensorParallelRowLinear):
        return module.in_features * world, module.out_features
    raise ValueError(type(module))


class LearningRateForParametrizator:
    def __init__(self, lr: float, names_to_modules: Dict[str, nn.Module]):
        self.lr = lr
        self.names_to_modules = names_to_modules

    def get_lr(self, param_name: str, module: nn.Module) -> float:
        for types, fn in self.MODULE_TO_PARAMETRIZE():
            if isinstance(module, types):
                return fn(param_name, module)
        raise Exception(f"Module {type(module)} with parameter {param_name} is not supported for per-parameter learning rates")


class LearningRateForSP(LearningRateForParametrizator):
    def MODULE_TO_PARAMETRIZE(self):
        return [((nn.Module,), lambda n, m: self.lr)]


class LearningRateForSpectralMup(LearningRateForParametrizator):
    """lr * fan_out / fan_in for matrices; base lr for norms and embeddings."""

    def MODULE_TO_PARAMETRIZE(self):
        return [
            (TensorParallelColumnLinear, self._get_mup_lr),
            (TensorParallelRowLinear, self._get_mup_lr),
            (_norm_types(), lambda n, m: self.lr),
            (TensorParallelEmbedding, lambda n, m: self.lr),
        ]

    def _get_mup_lr(self, param_name: str, module: nn.Module):
        fan_in, fan_out = _unsharded_fans(module)
        return self.lr * (fan_out / fan_in)
