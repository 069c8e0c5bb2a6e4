"""One fused data-parallel optimizer step over NVLink peer memory (ZeRO-1 or replicated optimizer).

Replaces, for a node-local data-parallel group on CUDA, the sequence
``NCCL reduce-scatter / all-reduce of fp32 grads -> grad-norm kernels -> clip multiply -> AdamW -> fp32->bf16 copy ->
NCCL all-gather of parameters`` (reference src/nanotron/optim/gradient_accumulator.py:128-156,
optim/clip_grads.py:54-97, optim/zero.py:94-120,217-252) by three in-tree kernels (``csrc/comm.cu``):

  barrier -> reduce-scatter by peer loads (+ 1/dp scale + sum of squares) -> [scalar norm all-reduce]
          -> AdamW on the master shard with bf16 results stored into every rank's parameter buffer -> barrier

Requirements: fp32 gradient accumulation (flat buffers), AdamW, all ranks of the dp group on one NVLink domain.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.optim.fused_adamw import FusedAdamW
from nanotron_b200.optim.zero import ZeroDistributedOptimizer


class FusedDataParallelStep:
    def __init__(self, allocator, grad_accumulator, optimizer, dp_pg, mp_pg, clip_grad: Optional[float]):
        from nanotron_b200.ops import native

        self.native = native
        self.alloc = allocator
        self.acc = grad_accumulator
        self.optimizer = optimizer
        self.base: FusedAdamW = optimizer.get_base_optimizer()
        self.dp_pg, self.mp_pg = dp_pg, mp_pg
        self.world = dp_pg.size()
        self.rank = dist.get_rank(dp_pg)
        self.clip_grad = clip_grad
        self.zero = optimizer.inherit_from(ZeroDistributedOptimizer)
        self.grad_sym = allocator.lookup(grad_accumulator._contiguous_fp32_grad_buffer)
        half = next(iter(grad_accumulator._contiguous_half_buffers.values()))
        self.param_sym = allocator.lookup(half)
        assert self.grad_sym is not None and self.param_sym is not None, "flat buffers are not in symmetric memory"
        layout = grad_accumulator.layout
        if self.zero:
            self.start, end = layout.shard_range(self.rank)
            self.n = end - self.start
        else:
            # replicated optimizer: every rank reduces its 1/dp slice and broadcasts it (all-reduce), then steps locally
            total = layout.total
            per = (total // self.world + 7) // 8 * 8
            self.start = min(self.rank * per, total)
            self.n = max(0, min(per, total - self.start))
        dev = allocator.device
        self.partials = torch.empty(native.lib().ntb_dp_num_partials(), dtype=torch.float32, device=dev)
        # flat ranges (inside this rank's reduced slice) of tied parameters whose squares another member of the tie group already counts
        self.duplicate_ranges = []
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_norm = None

    def exclude_tied_duplicates(self, named_params, world_rank: int):
        """A tied parameter (norm weights replicated over tp, embeddings tied across pipeline stages) has one gradient copy per
        member of its tie group.  The global norm counts it once, on the first rank of the group, as ``clip_grad_norm`` does
        (reference src/nanotron/optim/clip_grads.py:43-53): every other member records the part of the copy that lies in its
        reduced slice here, and ``step`` removes those squares from its partial sum before the all-reduce."""
        layout = self.acc.layout
        lo, hi = self.start, self.start + self.n
        self.duplicate_ranges = []
        for name, p in named_params:
            if not (p.requires_grad and getattr(p, "is_tied", False)):
                continue
            ranks = sorted(p.get_tied_info().global_ranks)
            if len(ranks) <= 1 or world_rank == ranks[0] or name not in layout.offsets:
                continue
            a, b = max(layout.offsets[name], lo), min(layout.offsets[name] + layout.numels[name], hi)
            if b > a:
                self.duplicate_ranges.append((a, b))

    def step(self):
        """Everything between the last backward and the next forward.  Returns the pre-clip gradient norm (or None)."""
        native, L = self.native, self.native.lib()
        stream = torch.cuda.current_stream().cuda_stream
        self.alloc.barrier()  # every rank finished accumulating its gradients
        rc = L.ntb_dp_reduce_scatter(self.grad_sym.ptrs, self.rank, self.world, self.start, self.n, 1.0 / self.world, 0 if self.zero else 1, self.partials.data_ptr(), self.sumsq.data_ptr(), stream)
        native._check(rc, "dp_reduce_scatter")
        total = self.sumsq.clone()
        if self.duplicate_ranges:
            flat = self.acc._contiguous_fp32_grad_buffer
            total -= torch.stack([flat[a:b].pow(2).sum() for a, b in self.duplicate_ranges]).sum()
        # every rank holds the squares of a disjoint slice: sum over dp, then over model-parallel ranks
        dist.all_reduce(total, group=self.dp_pg)
        if self.mp_pg is not None and self.mp_pg.size() > 1:
            dist.all_reduce(total, group=self.mp_pg)
        norm = total.sqrt()
        self.grad_norm = norm.squeeze()
        if self.clip_grad is not None:
            self.base.grad_scale = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0)
        if self.zero:
            self._adamw_allgather(stream)
        else:
            self.alloc.barrier()  # broadcast slices have landed everywhere
            self.optimizer.step()
        self.alloc.barrier()  # all parameter stores have landed before anyone starts the next forward
        return self.grad_norm

    def _adamw_allgather(self, stream):
        base = self.base
        if base._flat is None:
            base._flat = base._try_build_flat_plan()
            assert base._flat is not None, "fused ZeRO step needs the flat AdamW plan"
        plan = base._flat
        lrs = tuple(float(base.param_groups[gi]["lr"]) for gi in plan["seg_group"])
        if plan["lr_cache"] != lrs:
            plan["seg_lr"].copy_(torch.tensor(lrs, dtype=torch.float32), non_blocking=True)
            plan["lr_cache"] = lrs
        step_val = None
        for p, _ in plan["items"]:
            st = base.state[p]
            st["step"] += 1
            step_val = float(st["step"])
        g0 = base.param_groups[plan["seg_group"][0]]
        beta1, beta2 = g0["betas"]
        n = plan["p"].numel()
        assert n <= self.n and n % 8 == 0
        rc = self.native.lib().ntb_dp_adamw_allgather(
            plan["p"].data_ptr(), plan["g"].data_ptr(), plan["m"].data_ptr(), plan["v"].data_ptr(), self.param_sym.ptrs, self.rank, self.world,
            self.start, n, plan["seg_end"].data_ptr(), plan["seg_lr"].data_ptr(), plan["seg_wd"].data_ptr(), plan["seg_end"].numel(),
            beta1, beta2, g0["eps"], 1.0 - beta1**step_val, 1.0 - beta2**step_val,
            base.grad_scale.data_ptr() if base.grad_scale is not None else None, stream,
        )
        self.native._check(rc, "dp_adamw_allgather")
        for p, _ in plan["items"]:
            p._half_written = True
