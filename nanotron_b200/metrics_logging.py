"""Detailed per-layer statistics of weights and gradients (parity: reference src/nanotron/metrics_logging.py).

Level 0: global statistics only.  Level 1: per layer / per component (attention qkv and out projections, MLP
projections, norms) mean, std, min, max, L1/L2 norms, fraction of zeros and kurtosis, for weights and for their fp32
gradients.  Everything is computed on the device and gathered as one stacked tensor per call (one host sync).
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200.logging import get_logger
from nanotron_b200.parallel import ParallelContext

logger = get_logger(__name__)

STAT_NAMES = ["mean", "std", "min", "max", "l1", "l2", "zero_frac", "kurtosis"]


def compute_tensor_stats(t: torch.Tensor) -> torch.Tensor:
    """fp32 vector of STAT_NAMES for one tensor."""
    x = t.detach().float().reshape(-1)
    if x.numel() == 0:
        return torch.zeros(len(STAT_NAMES), device=t.device)
    mean = x.mean()
    c = x - mean
    var = (c * c).mean()
    std = var.sqrt()
    kurt = (c**4).mean() / (var * var + 1e-30)
    return torch.stack([mean, std, x.min(), x.max(), x.abs().sum(), (x * x).sum().sqrt(), (x == 0).float().mean(), kurt])


class MetricsLogger:
    """Collects metrics for the trainer's logger rank.  ``log_level`` 0 = global only, 1 = per layer."""

    COMPONENTS = {
        "attn/qkv_proj": r"\.attn\.(qkv_proj|query_key_value|qkv\.q|qkv\.kv)\.weight$",
        "attn/o_proj": r"\.attn\.(o_proj|dense|o)\.weight$",
        "mlp/gate_up_proj": r"\.(mlp|ff)\.(gate_up_proj|c_fc)\.weight$",
        "mlp/down_proj": r"\.(mlp|ff)\.(down_proj|c_proj)\.weight$",
        "input_layernorm": r"\.(input_layernorm|ln_1)\.weight$",
        "post_attention_layernorm": r"\.(post_attention_layernorm|ln_2)\.weight$",
        "router": r"\.mlp\.router\.weight$",
        "experts": r"\.mlp\.experts\.merged_(gate_up|down)_proj$",
    }

    def __init__(self, config):
        self.config = config
        ml = getattr(config, "metrics_logging", None)
        self.log_level = ml.log_level if ml is not None else 0
        self.log_detail_interval = ml.log_detail_interval if ml is not None else 10

    def _layer_of(self, name: str) -> Optional[int]:
        m = re.search(r"(?:^|\.)decoder\.(\d+)\.", name)
        return int(m.group(1)) if m else None

    def _component_of(self, name: str) -> Optional[str]:
        for comp, pat in self.COMPONENTS.items():
            if re.search(pat, name):
                return comp
        return None

    def collect_parameter_metrics(self, model: nn.Module, grad_accumulator=None) -> Dict[str, torch.Tensor]:
        keys: List[str] = []
        vals: List[torch.Tensor] = []
        named = list(model.get_named_params_with_correct_tied()) if hasattr(model, "get_named_params_with_correct_tied") else list(model.named_parameters())
        for name, p in named:
            layer, comp = self._layer_of(name), self._component_of(name)
            if comp is None:
                if "lm_head" in name:
                    prefix = "lm_head"
                elif "embedding" in name:
                    prefix = "token_embedding"
                elif "final_layer_norm" in name:
                    prefix = "final_layer_norm"
                else:
                    continue
            else:
                prefix = f"layer_{layer}/{comp}" if layer is not None else comp
            keys.append(f"weights/{prefix}")
            vals.append(compute_tensor_stats(p))
            grad = None
            if grad_accumulator is not None and name in grad_accumulator.fp32_grad_buffers:
                grad = grad_accumulator.get_grad_buffer(name)
            elif p.grad is not None:
                grad = p.grad
            if grad is not None:
                keys.append(f"grads/{prefix}")
                vals.append(compute_tensor_stats(grad))
        if not vals:
            return {}
        stacked = torch.stack(vals).cpu()  # single device -> host transfer
        out = {}
        for k, row in zip(keys, stacked):
            for stat, v in zip(STAT_NAMES, row):
                out[f"{k}/{stat}"] = v
        return out

    def collect_global_metrics(self, model: nn.Module, grad_accumulator=None) -> Dict[str, torch.Tensor]:
        ws = [p.detach().float().pow(2).sum() for p in model.parameters()]
        out = {"global/weights_l2": torch.stack(ws).sum().sqrt().cpu() if ws else torch.tensor(0.0)}
        if grad_accumulator is not None:
            out["global/grads_l2"] = grad_accumulator._contiguous_fp32_grad_buffer.float().pow(2).sum().sqrt().cpu()
        return out

    def collect_all_metrics(self, model: nn.Module, grad_accumulator=None, iteration_step: int = 0) -> Dict[str, torch.Tensor]:
        metrics = self.collect_global_metrics(model, grad_accumulator)
        if self.log_level >= 1 and iteration_step % self.log_detail_interval == 0:
            metrics.update(self.collect_parameter_metrics(model, grad_accumulator))
        return metrics
