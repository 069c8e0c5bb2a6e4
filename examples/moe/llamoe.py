"""LlaMoE: the model class of the mixture-of-experts example (capability parity: reference examples/moe/llamoe.py).

The decoder, the expert layers and the loss are the framework's (``Qwen2ForTraining`` builds ``Qwen2MoELayer`` blocks when the
model configuration carries a ``moe_config``); this class adds what a user model typically adds on top: its own weight-decay
policy and a per-expert load report fed by forward hooks on the routers.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from nanotron_b200.models.qwen import Qwen2ForTraining


class LlaMoEForTraining(Qwen2ForTraining):
    def __init__(self, config, parallel_context, parallel_config, random_states=None):
        super().__init__(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        self.expert_load: Dict[str, torch.Tensor] = {}
        self._hooks_installed = not getattr(config, "log_expert_load", False)

    def forward(self, *args, **kwargs):
        if not self._hooks_installed:
            # the blocks of this pipeline stage are only built after the constructor returns, so the routers are looked up here
            from nanotron_b200.nn.moe import Router

            for name, module in self.named_modules():
                if isinstance(module, Router):
                    module.register_forward_hook(self._make_hook(name, self.config.moe_config.num_experts))
            self._hooks_installed = True
        return super().forward(*args, **kwargs)

    def _make_hook(self, name: str, num_experts: int):
        def hook(module, args, output):
            # the router returns the chosen expert ids among its outputs: count them (no gradient, no synchronisation)
            ids = next((o for o in (output if isinstance(output, (tuple, list)) else output.values() if isinstance(output, dict) else [output])
                        if torch.is_tensor(o) and o.dtype in (torch.int32, torch.int64)), None)
            if ids is not None:
                counts = torch.bincount(ids.reshape(-1).long().clamp(0, num_experts - 1), minlength=num_experts).float()
                self.expert_load[name] = counts / counts.sum().clamp(min=1)

        return hook

    def expert_load_report(self) -> Dict[str, float]:
        """Largest token fraction any expert received in the last forward, per router (1 / num_experts is perfect balance)."""
        return {name: float(frac.max()) for name, frac in self.expert_load.items()}

    def get_named_params_without_weight_decay(self) -> List[str]:
        names = list(super().get_named_params_without_weight_decay())
        if not getattr(self.config, "router_weight_decay", False):
            names += [n for n, _ in self.named_parameters() if ".router." in n and n not in names]
        return names
