"""fp32 gradient accumulation and fp32 master weights over flat buffers.

Capability parity: reference src/nanotron/optim/gradient_accumulator.py:18-395.  Layout differences made for B200:

* ONE contiguous fp32 gradient buffer for all parameters; every half-precision parameter gets a ``main_grad`` view of
  its slice.  Weight-gradient GEMMs accumulate into ``main_grad`` in their epilogue, so for linears there is no bf16
  gradient tensor and no separate ``fp32 += bf16`` pass.  Parameters whose gradient comes from another op (norms,
  embeddings, routers) are folded in by a post-accumulate-grad hook that frees ``param.grad`` at once.
* ONE contiguous fp32 master buffer for the parameters (or parameter slices, under ZeRO-1) this rank optimises, so
  the optimizer, the gradient-norm and the fp32->bf16 write-back are single flat kernels.
* Data-parallel synchronisation is one collective on the flat buffer (all-reduce, or reduce-scatter when the
  optimizer state is sharded: implemented here, a ``NotImplementedError`` in the reference's DDP hook).
"""
from __future__ import annotations

import dataclasses
from abc import ABC, abstractmethod
from collections import OrderedDict
from contextlib import contextmanager
from typing import Callable, Dict, Iterator, Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.optim.flat_layout import ALIGN, FlatLayout, _round_up, alloc_flat, flatten_parameters
from nanotron_b200.parallel.parameters import NanotronParameter


class GradientAccumulator(ABC):
    fp32_grads_allreduce_handle: Optional[torch.futures.Future]

    @abstractmethod
    def __init__(self, named_parameters: Iterator[Tuple[str, NanotronParameter]]) -> None:
        ...

    @abstractmethod
    def backward(self, loss, grad_tensors=None):
        ...

    @abstractmethod
    def step(self):
        ...

    @abstractmethod
    def sync_gradients_across_dp(self, dp_pg: dist.ProcessGroup, reduce_op: dist.ReduceOp, reduce_scatter: bool):
        ...

    @abstractmethod
    def zero_grad(self):
        ...

    @abstractmethod
    def get_parameter_for_optimizer(self, name: str) -> NanotronParameter:
        ...

    @abstractmethod
    def get_grad_buffer(self, name: str) -> torch.Tensor:
        ...

    @abstractmethod
    def state_dict(self) -> Dict[str, torch.Tensor]:
        ...

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, torch.Tensor]):
        ...


class FP32GradientAccumulator(GradientAccumulator):
    def __init__(
        self,
        named_parameters: Iterator[Tuple[str, NanotronParameter]],
        grad_buckets_named_params: Optional[Iterator[Tuple[str, NanotronParameter]]] = None,
        fuse_wgrad_accumulation: bool = True,
        flat_shard_world: int = 1,
    ):
        """``named_parameters``: parameters this rank optimises (fp32 masters are created for them).
        ``grad_buckets_named_params``: parameters that need an fp32 gradient slot (default: the same ones; under
        ZeRO-1 it is all parameters of the model while ``named_parameters`` may be sliced later through
        :meth:`assign_param_offsets`)."""
        named_parameters = list(named_parameters)
        if grad_buckets_named_params is None:
            grad_buckets_named_params = named_parameters
        grad_buckets_named_params = [(n, p) for n, p in grad_buckets_named_params if p.requires_grad]
        named_parameters = [(n, p) for n, p in named_parameters if p.requires_grad]
        self._named = OrderedDict(named_parameters)
        self.fuse_wgrad_accumulation = fuse_wgrad_accumulation
        # ---- gradients
        self.layout = FlatLayout.build([(n, p.numel()) for n, p in grad_buckets_named_params], world=flat_shard_world)
        self.fp32_grad_buffers, self._contiguous_fp32_grad_buffer = self.build_grad_buffers(grad_buckets_named_params, self.layout)
        self.flat_shard_range = None
        self._grad_offsets = {n: d["offset"] for n, d in self.fp32_grad_buffers.items()}
        # half-precision parameters live in one flat buffer with the same layout, so the optimizer can write them back
        # (and ZeRO can all-gather them) as one contiguous range
        self._contiguous_half_buffers = {}
        if grad_buckets_named_params and len({p.dtype for _, p in grad_buckets_named_params}) == 1:
            self._contiguous_half_buffers = flatten_parameters(grad_buckets_named_params, self.layout)
        # ---- masters (whole parameters until assign_param_offsets narrows them)
        self.parameters: Dict[str, Dict[str, torch.Tensor]] = {}
        self._build_masters({n: (0, p.numel()) for n, p in named_parameters})
        self.param_name_to_offsets: Optional[Dict[str, Dict[int, Tuple[int, int]]]] = None
        self.dp_rank = 0
        self.fp32_grads_allreduce_handle = None
        self._is_accumulation_sync_step = False
        self._hooks = []
        self._attach_hooks(grad_buckets_named_params)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def build_grad_buffers(named_parameters, layout=None):
        named_parameters = list(named_parameters)
        if len(named_parameters) == 0:
            return {}, torch.zeros(0, dtype=torch.float32)
        device = named_parameters[0][1].device
        if layout is None:
            layout = FlatLayout.build([(n, p.numel()) for n, p in named_parameters])
        offsets = layout.offsets
        buf = alloc_flat(layout.total, torch.float32, device)
        out = OrderedDict()
        for name, p in named_parameters:
            view = buf[offsets[name] : offsets[name] + p.numel()].view(p.shape)
            out[name] = {"half": p, "fp32_grad": view, "offset": offsets[name]}
        return out, buf

    def _build_masters(self, name_to_range: Dict[str, Tuple[int, int]]):
        """(Re)create the flat fp32 master buffer holding ``param.view(-1)[start:end]`` for every listed name."""
        for d in self.parameters.values():
            d["fp32"].data = torch.empty(0)
        self.parameters = {}
        items = [(n, r) for n, r in name_to_range.items() if r[1] > r[0]]
        total, offs = 0, {}
        for n, (s, e) in items:
            offs[n] = total
            total += _round_up(e - s, ALIGN)
        device = next(iter(self._named.values())).device if self._named else torch.device("cpu")
        self._contiguous_fp32_master_buffer = torch.zeros(total, dtype=torch.float32, device=device)
        self._master_ranges = dict(items)
        with torch.no_grad():
            for n, (s, e) in items:
                half = self._named[n]
                flat = self._contiguous_fp32_master_buffer[offs[n] : offs[n] + (e - s)]
                flat.copy_(half.detach().reshape(-1)[s:e])
                master_data = flat.view(half.shape) if (s, e) == (0, half.numel()) else flat
                master = NanotronParameter(master_data, requires_grad=True)
                if isinstance(half, NanotronParameter):
                    # masters carry the same sharding / tying metadata as the parameter they shadow
                    setattr(master, NanotronParameter.NANOTRON_PARAMETER_METADATA_ATTRIBUTE_NAME, dict(half._meta))
                g = self.fp32_grad_buffers[n]["fp32_grad"].view(-1)[s:e]
                grad_view = g.view(half.shape) if (s, e) == (0, half.numel()) else g
                master.grad = grad_view
                self.parameters[n] = {"fp32": master, "half": half, "master_offset": offs[n], "grad_view": grad_view}

    def assign_param_offsets(self, param_name_to_offsets: Dict[str, Dict[int, Tuple[int, int]]], dp_rank: int):
        """ZeRO-1: keep masters only for the slice ``param_name_to_offsets[name][dp_rank]`` of every parameter."""
        self.param_name_to_offsets = param_name_to_offsets
        self.dp_rank = dp_rank
        if self.layout.world > 1:
            self.flat_shard_range = self.layout.shard_range(dp_rank)
        ranges = {}
        for n in self._named:
            per_rank = param_name_to_offsets.get(n, {})
            ranges[n] = tuple(per_rank.get(dp_rank, (0, 0)))
        self._build_masters(ranges)

    def _attach_hooks(self, named_parameters):
        for name, p in named_parameters:
            slot = self.fp32_grad_buffers[name]["fp32_grad"]
            if self.fuse_wgrad_accumulation:
                p.main_grad = slot

            def hook(param, slot=slot):
                if param.grad is not None:
                    slot.add_(param.grad)
                    param.grad = None

            self._hooks.append(p.register_post_accumulate_grad_hook(hook))

    # ------------------------------------------------------------------ training-step API
    def backward(self, loss, grad_tensors=None):
        """``loss``: a scalar, or a list of roots with matching ``grad_tensors`` (pipeline stages backpropagate from the activations
        they sent onwards, seeded with the gradients received for them)."""
        torch.autograd.backward(loss, grad_tensors)
        # gradients were folded into the fp32 buffer by hooks / GEMM epilogues

    @torch.no_grad()
    def step(self):
        """Write the updated fp32 masters back into the half-precision parameters."""
        for name, d in self.parameters.items():
            half, master = d["half"], d["fp32"]
            s, e = self._master_ranges[name]
            if getattr(master, "_half_written", False):
                master._half_written = False
                continue
            half.detach().view(-1)[s:e].copy_(master.detach().view(-1))

    def zero_grad(self):
        self._contiguous_fp32_grad_buffer.zero_()
        for d in self.fp32_grad_buffers.values():
            d["half"].grad = None
        # optimizers drop ``.grad`` in their own zero_grad: re-attach the views of the flat buffer to the masters
        for d in self.parameters.values():
            d["fp32"].grad = d["grad_view"]

    def get_parameter_for_optimizer(self, name: str) -> NanotronParameter:
        return self.parameters[name]["fp32"]

    def get_grad_buffer(self, name: str) -> torch.Tensor:
        return self.fp32_grad_buffers[name]["fp32_grad"]

    @contextmanager
    def no_sync(self):
        old = self._is_accumulation_sync_step
        self._is_accumulation_sync_step = False
        try:
            yield
        finally:
            self._is_accumulation_sync_step = old

    # ------------------------------------------------------------------ data-parallel synchronisation
    def sync_gradients_across_dp(self, dp_pg: dist.ProcessGroup, reduce_op: dist.ReduceOp, reduce_scatter: bool):
        """Average (or sum) the flat fp32 gradient buffer over ``dp_pg``.  ``reduce_scatter=True`` (ZeRO-1) only
        guarantees the slices this rank optimises to be reduced; it moves half the bytes of an all-reduce."""
        if dp_pg.size() == 1:
            return
        buf = self._contiguous_fp32_grad_buffer
        avg = reduce_op == dist.ReduceOp.AVG
        op = dist.ReduceOp.SUM if (avg and dist.get_backend(dp_pg) != "nccl") else reduce_op
        if reduce_scatter and self.param_name_to_offsets is not None and getattr(self, "flat_shard_range", None) is not None:
            s, e = self.flat_shard_range
            world = dp_pg.size()
            shard = (e - s)
            assert buf.numel() == shard * world, "flat gradient buffer must be padded to a multiple of the dp size"
            out = buf[s:e]
            if dist.get_backend(dp_pg) == "nccl":
                dist.reduce_scatter_tensor(out, buf, op=op, group=dp_pg)
            else:
                tmp = torch.empty_like(out)
                dist.reduce_scatter_tensor(tmp, buf, op=op, group=dp_pg)
                out.copy_(tmp)
            if avg and op != reduce_op:
                out.div_(world)
            return
        dist.all_reduce(buf, op=op, group=dp_pg)
        if avg and op != reduce_op:
            buf.div_(dp_pg.size())

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {name: d["fp32"].detach() for name, d in self.parameters.items()}

    def load_state_dict(self, state_dict: Dict[str, torch.Tensor]):
        assert set(state_dict.keys()) == set(self.parameters.keys()), f"fp32 master names mismatch: {set(state_dict) ^ set(self.parameters)}"
        with torch.no_grad():
            for name, d in self.parameters.items():
                d["fp32"].copy_(state_dict[name].view_as(d["fp32"]))
