"""Per-module "to-be-inspected" tensor logging (parity: reference src/nanotron/logging/logmixin.py).

A module deriving :class:`LogMixin` calls ``self.tbi_logger({"name": tensor})``; the root model,
deriving :class:`LoggingCollectorMixin`, gathers them with ``get_tbi_logs`` once per step.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


class LogMixin:
    def tbi_logger(self, tensors: Dict[str, torch.Tensor]):
        if not hasattr(self, "_tbi_logs"):
            self._tbi_logs: List[Dict[str, torch.Tensor]] = []
        self._tbi_logs.append({k: v.detach() for k, v in tensors.items()})

    def _get_tbi_logs(self):
        return getattr(self, "_tbi_logs", [])

    def _clear_tbi_logs(self):
        self._tbi_logs = []


class LoggingCollectorMixin:
    def get_tbi_logs(self, non_blocking: bool = False) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for name, module in self.named_modules():
            if isinstance(module, LogMixin):
                for i, entry in enumerate(module._get_tbi_logs()):
                    for k, v in entry.items():
                        key = f"{name}/{k}" if i == 0 else f"{name}/{k}/{i}"
                        out[key] = v.to("cpu", non_blocking=non_blocking)
        return out

    def clear_all_tbi_logs(self):
        for module in self.modules():
            if isinstance(module, LogMixin):
                module._clear_tbi_logs()
