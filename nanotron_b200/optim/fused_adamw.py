"""AdamW as a single multi-tensor kernel over fp32 parameters (state-dict compatible with ``torch.optim.AdamW``).

On CUDA all parameters of a group are updated by one launch of the in-tree kernel, which also (optionally) writes
the bf16 copy of each updated fp32 master into the model parameter, replacing the separate fp32->bf16 pass
(reference src/nanotron/optim/gradient_accumulator.py:255-267).  On CPU it runs the PyTorch formula.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from nanotron_b200.ops import reference as ref


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.half_targets: Dict[int, torch.Tensor] = {}  # id(master) -> flat half-precision destination view

    def set_half_target(self, master: torch.Tensor, half_view: torch.Tensor):
        """After each step also write ``master`` (cast) into ``half_view`` (same numel)."""
        assert master.numel() == half_view.numel()
        self.half_targets[id(master)] = half_view

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            ps, gs, ms, vs, halves = [], [], [], [], []
            beta1, beta2 = group["betas"]
            step_val = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["step"] += 1
                step_val = float(st["step"])
                ps.append(p)
                gs.append(p.grad)
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
                halves.append(self.half_targets.get(id(p)))
            if not ps:
                continue
            lr = float(group["lr"]) if not isinstance(group["lr"], torch.Tensor) else float(group["lr"].item())
            if ps[0].is_cuda and ps[0].dtype == torch.float32:
                from nanotron_b200 import ops
                from nanotron_b200.ops import native

                if ops.get_mode() != "torch":
                    native.multi_tensor_adamw(ps, gs, ms, vs, halves, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val)
                    for p, h in zip(ps, halves):
                        if h is not None:
                            p._half_written = True
                    continue
            for p, g, m, v, h in zip(ps, gs, ms, vs, halves):
                if p.dtype == torch.float32:
                    ref.adamw_step(p, g.float(), m, v, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val)
                else:
                    pf, mf, vf = p.float(), m.float(), v.float()
                    ref.adamw_step(pf, g.float(), mf, vf, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val)
                    p.copy_(pf), m.copy_(mf), v.copy_(vf)
                if h is not None:
                    h.copy_(p.view(-1))
                    p._half_written = True
        return loss
