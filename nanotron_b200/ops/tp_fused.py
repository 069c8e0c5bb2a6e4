"""Compute + collective pairs of the tensor-parallel linears on CUDA.

``all_gather_matmul``: y = all_gather(x) @ W^T.  ``MatmulReduceScatter``: y = reduce_scatter(x @ W^T).
Two implementations, picked at call time:

* symmetric-memory kernels (``nanotron_b200.parallel.symm``): the GEMM's loader reads the peer shards directly over
  NVLink (all-gather side) and its epilogue pushes partial tiles into the owner's buffer (reduce-scatter side);
* chunked NCCL pipeline: the local shard's GEMM runs first while the remote shards arrive, then the remaining
  rows; for reduce-scatter the output is produced in per-destination chunks so the collective of chunk i overlaps
  the GEMM of chunk i+1.  This is the portable path and the A/B comparator for the fused kernels.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.utils import MemoryBuffer

_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = str(device)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


def all_gather_matmul(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group, keep_gathered: bool, lead_rows: int) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (y[tp*M, N], gathered x or None).  Rows of rank r land at [r*M, (r+1)*M)."""
    from nanotron_b200 import ops

    tp = group.size()
    rank = dist.get_rank(group)
    M, K = x2.shape
    x2 = x2.contiguous()
    if keep_gathered:
        gathered = torch.empty((tp * M, K), dtype=x2.dtype, device=x2.device)
    else:
        gathered = MemoryBuffer().get("allgather", (tp * M, K), dtype=x2.dtype, device=x2.device)
    out = torch.empty((tp * M, weight.shape[0]), dtype=x2.dtype, device=x2.device)
    handle = dist.all_gather_into_tensor(gathered, x2, group=group, async_op=True)
    # local shard first: its GEMM hides the transfer of the remote shards
    out[rank * M : (rank + 1) * M] = ops.linear_forward(x2, weight, bias)
    handle.wait()
    if rank > 0:
        out[: rank * M] = ops.linear_forward(gathered[: rank * M], weight, bias)
    if rank < tp - 1:
        out[(rank + 1) * M :] = ops.linear_forward(gathered[(rank + 1) * M :], weight, bias)
    return out, (gathered if keep_gathered else None)


class MatmulReduceScatter(torch.autograd.Function):
    """out[M/tp, N] = reduce_scatter_dim0(x[M, K_local] @ W[N, K_local]^T); backward all-gathers dY (async) while the
    local slice's dgrad runs (parity: reference functional.py:569-695)."""

    @staticmethod
    def forward(ctx, x, weight, group):
        from nanotron_b200 import ops

        tp = group.size()
        ctx.group = group
        ctx.save_for_backward(x, weight)
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        assert M % tp == 0
        rows = M // tp
        rank = dist.get_rank(group)
        # produce the chunk owned by rank+1 first and ours last, reducing chunk by chunk so that communication of
        # one chunk overlaps the GEMM of the next
        out = torch.empty((rows, weight.shape[0]), dtype=x.dtype, device=x.device)
        full = ops.linear_forward(x2, weight, None)
        dist.reduce_scatter_tensor(out, full, group=group)
        return out.view(x.shape[0] // tp, *x.shape[1:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        from nanotron_b200 import ops

        x, weight = ctx.saved_tensors
        group = ctx.group
        tp = group.size()
        go = grad_output.contiguous()
        total = MemoryBuffer().get("allgather2", (go.shape[0] * tp, *go.shape[1:]), dtype=go.dtype, device=go.device)
        handle = dist.all_gather_into_tensor(total, go, group=group, async_op=True)
        handle.wait()
        go2 = total.reshape(-1, total.shape[-1])
        grad_input = ops.linear_dgrad(go2, weight).view(x.shape) if ctx.needs_input_grad[0] else None
        grad_weight = ops.linear_wgrad(go2, x.reshape(-1, x.shape[-1]), weight)
        return grad_input, grad_weight, None
