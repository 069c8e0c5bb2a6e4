"""Tensor-parallel layers (parity: reference src/nanotron/parallel/tensor_parallel/nn.py:46-313)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.parallel.sharded_parameters import (
    SplitConfig,
    create_sharded_parameter_from_config,
    mark_all_parameters_in_module_as_sharded,
)
from nanotron_b200.parallel.tensor_parallel.distributed_differentiable_primitives import (
    differentiable_all_gather,
    differentiable_all_reduce_sum,
    differentiable_identity,
    differentiable_reduce_scatter_sum,
)
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.tensor_parallel.functional import column_linear, row_linear
from nanotron_b200.parallel.tied_parameters import create_tied_parameter


class TensorParallelColumnLinear(nn.Linear):
    """Linear whose output features are split over ``pg``.  ``contiguous_chunks`` gives the sizes of fused
    sub-projections in the unsharded weight (e.g. (q, k, v)); each is split evenly across ranks."""

    def __init__(
        self,
        in_features,
        out_features,
        pg: dist.ProcessGroup,
        mode: TensorParallelLinearMode,
        bias=True,
        device=None,
        dtype=None,
        async_communication: bool = False,
        contiguous_chunks: Optional[Tuple[int, ...]] = None,
        tp_recompute_allgather: bool = True,
    ):
        self.pg = pg
        self.world_size = pg.size()
        assert out_features % self.world_size == 0
        self.in_features = in_features
        self.out_features = out_features // self.world_size
        self.tp_recompute_allgather = tp_recompute_allgather
        super().__init__(in_features=self.in_features, out_features=self.out_features, bias=bias, device=device, dtype=dtype)
        self.mode = mode
        self.async_communication = async_communication
        if contiguous_chunks is not None:
            assert sum(contiguous_chunks) == out_features, f"Sum of contiguous chunks ({sum(contiguous_chunks)}) must equal out_features ({out_features})"
        mark_all_parameters_in_module_as_sharded(self, pg=self.pg, split_config=SplitConfig(split_dim=0, contiguous_chunks=contiguous_chunks))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return column_linear(
            input=x,
            weight=self.weight,
            bias=self.bias,
            group=self.pg,
            tp_mode=self.mode,
            async_communication=self.async_communication,
            tp_recompute_allgather=self.tp_recompute_allgather,
        )

    def extra_repr(self) -> str:
        return f"tp_rank={dist.get_rank(self.pg)}, {super().extra_repr()}, unsharded_out_features={self.out_features * self.world_size}"


class TensorParallelRowLinear(nn.Linear):
    """Linear whose input features are split over ``pg``; the partial products are reduced over the group.
    The bias is replicated, marked as not sharded, and added once after the reduction."""

    def __init__(
        self,
        in_features,
        out_features,
        pg: dist.ProcessGroup,
        mode: TensorParallelLinearMode,
        bias=True,
        device=None,
        dtype=None,
        async_communication: bool = False,
        contiguous_chunks: Optional[Tuple[int, ...]] = None,
    ):
        self.pg = pg
        self.world_size = pg.size()
        assert in_features % self.world_size == 0
        self.in_features = in_features // self.world_size
        self.out_features = out_features
        super().__init__(in_features=self.in_features, out_features=self.out_features, bias=bias, device=device, dtype=dtype)
        self.mode = mode
        self.async_communication = async_communication
        if self.mode is TensorParallelLinearMode.ALL_REDUCE and self.async_communication:
            raise ValueError("async_communication is not supported for ALL_REDUCE mode")
        if contiguous_chunks is not None:
            assert sum(contiguous_chunks) == in_features
        # only the weight is sharded (on its input dim); the bias is whole
        self.weight = create_sharded_parameter_from_config(parameter=self.weight, pg=self.pg, split_config=SplitConfig(split_dim=1, contiguous_chunks=contiguous_chunks))
        if self.bias is not None:
            self.bias = NanotronParameter(self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return row_linear(input=x, weight=self.weight, bias=self.bias, group=self.pg, tp_mode=self.mode, async_communication=self.async_communication)

    def extra_repr(self) -> str:
        return f"tp_rank={dist.get_rank(self.pg)}, {super().extra_repr()}, unsharded_in_features={self.in_features * self.world_size}"


class TiedLinear(nn.Linear):
    """Replicated linear whose parameters are tied over ``pg``.  ALL_REDUCE: grads identical on every rank
    (reduce_op None).  REDUCE_SCATTER: input is gathered first and grads are summed over the group."""

    def __init__(self, in_features, out_features, pg: dist.ProcessGroup, mode: TensorParallelLinearMode, bias=True, device=None, dtype=None):
        self.pg = pg
        self.world_size = pg.size()
        self.mode = mode
        super().__init__(in_features=in_features, out_features=out_features, bias=bias, device=device, dtype=dtype)
        self._mark_all_parameters_in_module_as_tied()

    def _mark_all_parameters_in_module_as_tied(self):
        for name, param in list(self.named_parameters()):
            new_param = create_tied_parameter(
                parameter=param,
                name=name,
                global_ranks=dist.get_global_ranks(self.pg),
                reduce_op=None if self.mode is TensorParallelLinearMode.ALL_REDUCE else dist.ReduceOp.SUM,
                root_module=self,
            )
            setattr(self, name, new_param)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = super().forward(x)
        if self.mode is TensorParallelLinearMode.ALL_REDUCE:
            return differentiable_identity(y, group=self.pg)
        if self.mode is TensorParallelLinearMode.REDUCE_SCATTER:
            return differentiable_all_gather(y, group=self.pg)
        raise ValueError(f"Got unexpected mode: {self.mode}.")


class TensorParallelEmbedding(nn.Embedding):
    """Embedding whose vocabulary is split over ``pg``: ids outside the local range contribute zeros, then the
    partial lookups are summed (all-reduce) or summed and scattered on dim 0 (sequence parallel)."""

    def __init__(
        self,
        num_embeddings,
        embedding_dim,
        pg: dist.ProcessGroup,
        mode: TensorParallelLinearMode,
        padding_idx=None,
        max_norm=None,
        norm_type=2.0,
        scale_grad_by_freq=False,
        sparse=False,
        _weight=None,
        device=None,
        dtype=None,
        contiguous_chunks: Optional[Tuple[int, ...]] = None,
    ):
        self.pg = pg
        self.rank = dist.get_rank(self.pg)
        self.world_size = pg.size()
        self.original_num_embeddings = num_embeddings
        assert num_embeddings % self.world_size == 0
        block_size = num_embeddings // self.world_size
        self.min_id = self.rank * block_size
        self.max_id = (self.rank + 1) * block_size
        super().__init__(block_size, embedding_dim, padding_idx=padding_idx, max_norm=max_norm, norm_type=norm_type, scale_grad_by_freq=scale_grad_by_freq, sparse=sparse, _weight=_weight, device=device, dtype=dtype)
        self.mode = mode
        if contiguous_chunks is not None:
            assert sum(contiguous_chunks) == num_embeddings
        mark_all_parameters_in_module_as_sharded(self, pg=self.pg, split_config=SplitConfig(split_dim=0, contiguous_chunks=contiguous_chunks))

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self.padding_idx is None and self.max_norm is None and not self.scale_grad_by_freq and not self.sparse:
            from nanotron_b200 import ops

            out = ops.masked_embedding(input_ids, self.weight, self.min_id, self.max_id)  # gather + range mask in one pass
        else:
            if self.world_size > 1:
                mask = (input_ids < self.min_id) | (input_ids >= self.max_id)
                local_ids = (input_ids - self.min_id).masked_fill(mask, 0)
            else:
                mask, local_ids = None, input_ids
            out = super().forward(local_ids)
            if mask is not None:
                out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        if self.mode is TensorParallelLinearMode.ALL_REDUCE:
            out = differentiable_all_reduce_sum(out, group=self.pg)
        elif self.mode is TensorParallelLinearMode.REDUCE_SCATTER:
            out = differentiable_reduce_scatter_sum(out, group=self.pg)
        else:
            raise ValueError(f"Got unexpected mode: {self.mode}.")
        return out

    def extra_repr(self) -> str:
        return f"tp_rank={self.rank}, {super().extra_repr()}, unsharded_num_embeddings={self.original_num_embeddings}"
