"""One fused data-parallel optimizer step over NVLink peer memory (ZeRO-1 or replicated optimizer).

Replaces, for a node-local data-parallel group on CUDA, the sequence
``NCCL reduce-scatter / all-reduce of fp32 grads -> grad-norm kernels -> clip multiply -> AdamW -> fp32->bf16 copy ->
NCCL all-gather of parameters`` (reference src/nanotron/optim/gradient_accumulator.py:128-156,
optim/clip_grads.py:54-97, optim/zero.py:94-120,217-252) by three in-tree kernels (``csrc/comm.cu``):

  barrier -> reduce-scatter by peer loads (+ 1/dp scale + sum of squares) -> [scalar norm all-reduce]
          -> AdamW on the master shard with bf16 results stored into every rank's parameter buffer -> barrier

Requirements: fp32 gradient accumulation (flat buffers), AdamW, all ranks of the dp group on one NVLink domain.

Overlap with the backward pass (``install_overlap``): the flat buffer is cut into one bucket per pipeline block (decoder layer,
lm head, ...).  During the LAST micro-batch's backward, the moment a block's input gradient exists all of the block's parameter
gradients are final, so a side stream runs, for that bucket, a device barrier over the dp group (every rank finished the bucket)
followed by the reduce-scatter of the part of it that falls into this rank's shard, on a bounded number of SMs, while the main
stream keeps differentiating the earlier layers (the reference overlaps its bucketed all-reduce from a DDP hook:
src/nanotron/optim/gradient_accumulator.py:322-394).  Parameters tied across ranks are left out of the early buckets because
their tie-group sum runs after the backward; ``step`` reduces whatever is left, then AdamW + all-gather as before.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Dict, List, Optional, Tuple

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
        # overlap with backward (see install_overlap)
        self.buckets: List[List[Tuple[int, int]]] = []  # per bucket: sub-ranges of this rank's slice, tied parameters excluded
        self.done: List[Tuple[int, int]] = []           # sub-ranges already reduced in this step
        self.armed = False
        self.launched = set()
        self.side = None
        self.side_done = None
        self.sumsq_acc = torch.zeros(1, dtype=torch.float32, device=dev)
        self.overlap_blocks = 48  # SMs the early reduce-scatter may occupy next to the backward GEMMs
        self.bucket_flags = None
        self.bucket_epoch = 0
        self.overlapped_elems = 0
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

    # ------------------------------------------------------------------ overlap with the backward pass
    def install_overlap(self, model, named_params) -> int:
        """Cut the flat buffer into one bucket per ``PipelineBlock`` of ``model`` and hook the blocks so that a bucket is reduced as
        soon as the last micro-batch's backward has left it.  Returns the number of buckets that can go early on this rank."""
        from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

        layout = self.acc.layout
        lo, hi = self.start, self.start + self.n
        param_names = {id(p): n for n, p in named_params}
        self.buckets = []
        self.side = torch.cuda.Stream(device=self.alloc.device)
        self.side_done = torch.cuda.Event()
        self.bucket_flags = self.alloc.zeros(32, torch.int32)
        count = 0
        for block in (m for m in model.modules() if isinstance(m, PipelineBlock) and hasattr(m, "pp_block")):
            runs: List[Tuple[int, int]] = []
            for p in block.pp_block.parameters():
                name = param_names.get(id(p))
                if name is None or name not in layout.offsets or not p.requires_grad:
                    continue
                if getattr(p, "is_tied", False) and len(p.get_tied_info().global_ranks) > 1:
                    continue  # summed over its tie group after the backward: reduced in step()
                a, b = max(layout.offsets[name], lo), min(layout.offsets[name] + layout.numels[name], hi)
                a = (a + 3) // 4 * 4
                b = b // 4 * 4
                if b > a:
                    if runs and runs[-1][1] == a:
                        runs[-1] = (runs[-1][0], b)
                    else:
                        runs.append((a, b))
            idx = len(self.buckets)
            self.buckets.append(runs)
            count += bool(runs)
            block.pp_block.register_forward_pre_hook(self._make_pre_hook(idx), with_kwargs=True)
        return count

    def _make_pre_hook(self, idx: int):
        def pre_hook(module, args, kwargs):
            if not torch.is_grad_enabled():
                return None
            for v in list(args) + list(kwargs.values()):
                if isinstance(v, torch.Tensor) and v.requires_grad:
                    v.register_hook(lambda g, idx=idx: self._bucket_ready(idx))
                    break
            return None

        return pre_hook

    @contextlib.contextmanager
    def prepare_last_backward(self):
        """Entered by the pipeline engine around the backward of the last micro-batch of a step."""
        self.armed = True
        try:
            yield
        finally:
            self.armed = False

    def _bucket_ready(self, idx: int):
        """Autograd reached the input of block ``idx`` during the last backward: every gradient of the block is final on this rank."""
        if not self.armed or idx in self.launched:
            return None  # (a block's forward can run twice under activation recompute: its bucket still goes once)
        self.launched.add(idx)
        main = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        L = self.native.lib()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            # every rank of the group passes here for every bucket, in the same order: a barrier of its own flag words
            self.bucket_epoch += 1
            rc = L.ntb_symm_barrier(self.bucket_flags.ptrs, self.rank, self.world, self.bucket_epoch, self.alloc.wait_limit_ns, self.alloc.status.data_ptr(), self.side.cuda_stream)
            self.native._check(rc, "symm_barrier")
            for a, b in self.buckets[idx]:
                rc = L.ntb_dp_reduce_scatter_range(self.grad_sym.ptrs, self.rank, self.world, a, b - a, 1.0 / self.world, 0 if self.zero else 1, self.partials.data_ptr(), self.sumsq_acc.data_ptr(), self.overlap_blocks, self.side.cuda_stream)
                self.native._check(rc, "dp_reduce_scatter_range")
                self.done.append((a, b))
                self.overlapped_elems += b - a
            self.side_done.record(self.side)
        return None

    def _remaining(self) -> List[Tuple[int, int]]:
        """Sub-ranges of this rank's slice that no early bucket covered."""
        out, cur = [], self.start
        for a, b in sorted(self.done):
            if a > cur:
                out.append((cur, a))
            cur = max(cur, b)
        if cur < self.start + self.n:
            out.append((cur, self.start + self.n))
        return out

    def step(self):
        """Everything between the last backward and the next forward.  Returns the pre-clip gradient norm (or None)."""
        native, L = self.native, self.native.lib()
        main = torch.cuda.current_stream()
        stream = main.cuda_stream
        self.alloc.barrier()  # every rank finished accumulating its gradients
        if self.done:
            main.wait_event(self.side_done)  # the early buckets are reduced; their squares are in sumsq_acc
            for a, b in self._remaining():
                rc = L.ntb_dp_reduce_scatter_range(self.grad_sym.ptrs, self.rank, self.world, a, b - a, 1.0 / self.world, 0 if self.zero else 1, self.partials.data_ptr(), self.sumsq_acc.data_ptr(), L.ntb_dp_num_partials(), stream)
                native._check(rc, "dp_reduce_scatter_range")
            total = self.sumsq_acc.clone()
            self.sumsq_acc.zero_()
            self.done = []
        else:
            rc = L.ntb_dp_reduce_scatter(self.grad_sym.ptrs, self.rank, self.world, self.start, self.n, 1.0 / self.world, 0 if self.zero else 1, self.partials.data_ptr(), self.sumsq.data_ptr(), stream)
            native._check(rc, "dp_reduce_scatter")
            total = self.sumsq.clone()
        self.launched = set()
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
