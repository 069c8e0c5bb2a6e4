"""AdamW over fp32 parameters (state-dict compatible with ``torch.optim.AdamW``).

On CUDA, when every parameter is a slice of ONE contiguous fp32 master buffer (what the fp32 gradient accumulator
builds) and its gradient / half-precision twin sit at a constant offset in their own flat buffers, the whole
optimizer step is a single launch of the in-tree flat kernel: gradient scaling (clipping coefficient read on the
device), AdamW, and the bf16 write-back of the updated weights, replacing the separate fp32->bf16 pass of the
reference (reference src/nanotron/optim/gradient_accumulator.py:255-267).  The ``exp_avg`` / ``exp_avg_sq`` states
are views of two flat buffers with the same layout.  Otherwise (CPU, or scattered tensors) it runs per tensor.
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
        self.grad_scale: Optional[torch.Tensor] = None  # optional device scalar multiplied into every gradient
        self._flat = None  # cached flat plan
        self._flat_failed = False

    def set_half_target(self, master: torch.Tensor, half_view: torch.Tensor):
        """After each step also write ``master`` (cast) into ``half_view`` (same numel)."""
        assert master.numel() == half_view.numel()
        self.half_targets[id(master)] = half_view
        self._flat = None

    # ------------------------------------------------------------------ state
    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["step"] = torch.zeros((), dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    def _try_build_flat_plan(self):
        """All params must tile one contiguous fp32 range in address order, with constant grad / half offsets."""
        items = []
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                if p.grad is None or p.numel() == 0:
                    continue
                items.append((p, gi))
        if not items or not items[0][0].is_cuda or any(p.dtype != torch.float32 or not p.is_contiguous() for p, _ in items):
            return None
        items.sort(key=lambda it: it[0].data_ptr())
        first = items[0][0]
        base = first.data_ptr()
        gbase = first.grad.data_ptr()
        h0 = self.half_targets.get(id(first))
        use_half = h0 is not None
        hbase = h0.data_ptr() if use_half else 0
        storage_end = first.untyped_storage().data_ptr() + first.untyped_storage().nbytes()
        segs = []
        cursor = 0  # elements from base
        for p, gi in items:
            off = (p.data_ptr() - base) // 4
            if (p.data_ptr() - base) % 4 or off < cursor or off - cursor >= 128:
                return None  # gaps larger than the alignment padding: not one flat range
            g = p.grad
            if g.dtype != torch.float32 or not g.is_contiguous() or g.data_ptr() - gbase != p.data_ptr() - base:
                return None
            h = self.half_targets.get(id(p))
            if use_half != (h is not None):
                return None
            if use_half and (h.dtype != torch.bfloat16 or (h.data_ptr() - hbase) * 2 != p.data_ptr() - base):
                return None
            cursor = off + p.numel()
            segs.append((cursor, gi))
        total = (cursor + 3) // 4 * 4
        if base + total * 4 > storage_end or base % 16 or gbase % 16 or (use_half and hbase % 8):
            return None
        # merge neighbouring segments of the same group; padding elements between parameters take the hyper-parameters
        # of the following segment (they are zeros and stay zeros: zero grad, zero weight)
        merged = []
        for end, gi in segs:
            if merged and merged[-1][1] == gi:
                merged[-1] = (end, gi)
            else:
                merged.append((end, gi))
        merged[-1] = (total, merged[-1][1])
        dev = first.device
        flat_p = torch.as_strided(first, (total,), (1,), storage_offset=first.storage_offset())
        flat_g = torch.as_strided(first.grad, (total,), (1,), storage_offset=first.grad.storage_offset())
        flat_h = torch.as_strided(h0, (total,), (1,), storage_offset=h0.storage_offset()) if use_half else None
        # states: adopt existing values, then re-home them in flat buffers
        flat_m = torch.zeros(total, dtype=torch.float32, device=dev)
        flat_v = torch.zeros(total, dtype=torch.float32, device=dev)
        for p, _ in items:
            st = self._init_state(p)
            off = (p.data_ptr() - base) // 4
            for key, flat in (("exp_avg", flat_m), ("exp_avg_sq", flat_v)):
                view = flat[off : off + p.numel()].view(p.shape)
                view.copy_(st[key].to(dev))
                st[key] = view
        return {
            "p": flat_p, "g": flat_g, "h": flat_h, "m": flat_m, "v": flat_v, "items": items,
            "seg_end": torch.tensor([e for e, _ in merged], dtype=torch.int64, device=dev),
            "seg_group": [gi for _, gi in merged],
            "seg_lr": torch.empty(len(merged), dtype=torch.float32, device=dev),
            "seg_wd": torch.tensor([float(self.param_groups[gi]["weight_decay"]) for _, gi in merged], dtype=torch.float32, device=dev),
            "lr_cache": None,
        }

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        from nanotron_b200 import ops

        first = next((p for g in self.param_groups for p in g["params"]), None)
        if first is not None and first.is_cuda and ops.get_mode() != "torch" and not self._flat_failed:
            if self._flat is None:
                self._flat = self._try_build_flat_plan()
                self._flat_failed = self._flat is None
            if self._flat is not None:
                self._flat_step()
                return loss
        self._per_tensor_step()
        return loss

    def _flat_step(self):
        from nanotron_b200.ops import native

        plan = self._flat
        lrs = tuple(float(self.param_groups[gi]["lr"]) for gi in plan["seg_group"])
        if plan["lr_cache"] != lrs:
            plan["seg_lr"].copy_(torch.tensor(lrs, dtype=torch.float32), non_blocking=True)
            plan["lr_cache"] = lrs
        step_val = None
        for p, _ in plan["items"]:
            st = self.state[p]
            st["step"] += 1
            step_val = float(st["step"])
        g0 = self.param_groups[plan["seg_group"][0]]
        beta1, beta2 = g0["betas"]
        native.adamw_flat(plan["p"], plan["g"], plan["m"], plan["v"], plan["h"], plan["seg_end"], plan["seg_lr"], plan["seg_wd"], beta1, beta2, g0["eps"], step_val, self.grad_scale)
        if plan["h"] is not None:
            for p, _ in plan["items"]:
                p._half_written = True

    def _per_tensor_step(self):
        from nanotron_b200 import ops

        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr = float(group["lr"])
            ps, gs, ms, vs, halves = [], [], [], [], []
            step_val = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                step_val = float(st["step"])
                ps.append(p), gs.append(p.grad), ms.append(st["exp_avg"]), vs.append(st["exp_avg_sq"]), halves.append(self.half_targets.get(id(p)))
            if not ps:
                continue
            if ps[0].is_cuda and ps[0].dtype == torch.float32 and ops.get_mode() != "torch" and self.grad_scale is None:
                from nanotron_b200.ops import native

                native.multi_tensor_adamw(ps, gs, ms, vs, halves, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val)
            else:
                scale = float(self.grad_scale) if self.grad_scale is not None else 1.0
                for p, g, m, v, h in zip(ps, gs, ms, vs, halves):
                    if p.dtype == torch.float32:
                        ref.adamw_step(p, g.float(), m, v, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val, grad_scale=scale)
                    else:
                        pf, mf, vf = p.float(), m.float(), v.float()
                        ref.adamw_step(pf, g.float(), mf, vf, lr, beta1, beta2, group["eps"], group["weight_decay"], step_val, grad_scale=scale)
                        p.copy_(pf), m.copy_(mf), v.copy_(vf)
                    if h is not None:
                        h.copy_(p.view(-1))
            for p, h in zip(ps, halves):
                if h is not None:
                    p._half_written = True
