"""Tensor-parallel linear algebra: column / row linears (with optional sequence parallelism) and the
vocabulary-parallel cross entropy.

Behavioural parity with reference src/nanotron/parallel/tensor_parallel/functional.py:31-718, organised
differently: one autograd Function per linear, parameterised by a *communication plan* instead of one class
per (mode x async) combination.

* sync plan: collective, then GEMM (or GEMM, then collective).
* async plan (``async_communication=True``): on CUDA the all-gather -> GEMM and GEMM -> reduce-scatter pairs are
  issued as chunked pipelines on a side stream so the NVLink transfer of chunk i+1 overlaps the GEMM of chunk i;
  when the symmetric-memory kernels are available (see ``nanotron_b200.parallel.symm``) the pair is one fused
  kernel.  On CPU/gloo async handles are used.

Every GEMM goes through :func:`nanotron_b200.ops.linear_forward` / ``linear_dgrad`` / ``linear_wgrad`` so the
tcgen05 kernels replace the library call in one place.  Weight gradients can accumulate straight into an fp32
``main_grad`` buffer attached to the weight (set by the gradient accumulator), which removes the per-parameter
``fp32 += bf16`` pass the reference does (reference src/nanotron/optim/gradient_accumulator.py:206-239).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200 import ops
from nanotron_b200.parallel.tensor_parallel.distributed_differentiable_primitives import (
    differentiable_all_reduce_sum,
    differentiable_identity,
)
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.utils import MemoryBuffer


# ----------------------------------------------------------------------------- collectives helpers
def _all_gather_dim0(x: torch.Tensor, group, buffer_name: Optional[str] = None) -> torch.Tensor:
    if group is None or group.size() == 1:
        return x
    x = x.contiguous()
    shape = (x.shape[0] * group.size(), *x.shape[1:])
    if buffer_name is not None:
        out = MemoryBuffer().get(buffer_name, shape, dtype=x.dtype, device=x.device)
    else:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_dim0(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or group.size() == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] // group.size(), *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, op=dist.ReduceOp.SUM, group=group)
    return out


def _flatten2d(x: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, ...]]:
    lead = tuple(x.shape[:-1])
    return x.reshape(-1, x.shape[-1]), lead


class _TPLinear(torch.autograd.Function):
    """y = gather?(x) @ W^T (+b), then reduce?(y).

    ``pre``  in {"none", "all_gather"}           : collective applied to the input on dim 0
    ``post`` in {"none", "all_reduce", "reduce_scatter"} : collective applied to the output
    Backward applies the transposed collectives: all_gather<->reduce_scatter, identity<->all_reduce.
    ``input_grad_reduce``: for column-linear in ALL_REDUCE mode the input gradient is all-reduced.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, group, pre: str, post: str, input_grad_reduce: bool, async_comm: bool, recompute_allgather: bool):
        ctx.group, ctx.pre, ctx.post = group, pre, post
        ctx.input_grad_reduce, ctx.async_comm, ctx.recompute_allgather = input_grad_reduce, async_comm, recompute_allgather
        ctx.use_bias = bias is not None
        tp = group.size() if group is not None else 1
        x2, lead = _flatten2d(x)
        ctx.x_shape = x.shape
        if pre == "all_gather" and tp > 1:
            assert x.dim() >= 2
            if async_comm and x.is_cuda:
                out2, gathered = ops.tp_fused.all_gather_matmul(x2, weight, bias, group, keep_gathered=not recompute_allgather, lead_rows=x.shape[0])
            else:
                gathered = _all_gather_dim0(x, group, buffer_name="allgather" if recompute_allgather else None)
                g2, lead = _flatten2d(gathered)
                out2 = ops.linear_forward(g2, weight, bias)
            lead = (x.shape[0] * tp, *x.shape[1:-1])
            saved_in = x if recompute_allgather else gathered
        else:
            out2 = ops.linear_forward(x2, weight, bias)
            saved_in = x
        out = out2.view(*lead, weight.shape[0])
        if tp > 1 and post == "all_reduce":
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        elif tp > 1 and post == "reduce_scatter":
            out = _reduce_scatter_dim0(out, group)
        ctx.save_for_backward(saved_in, weight)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        saved_in, weight = ctx.saved_tensors
        group, pre, post = ctx.group, ctx.pre, ctx.post
        tp = group.size() if group is not None else 1
        grad_output = grad_output.contiguous()
        handle = None
        # ---- transpose of the output collective
        if tp > 1 and post == "reduce_scatter":
            grad_output = _all_gather_dim0(grad_output, group, buffer_name="allgather2")
        # (all_reduce forward -> identity backward)
        # ---- recover the full input if it was gathered in forward
        fused_ok = ctx.async_comm and grad_output.is_cuda and tp > 1
        if pre == "all_gather" and tp > 1 and ctx.recompute_allgather:
            xs = saved_in.contiguous()
            total = None
            if fused_ok:
                g = ops.tp_fused.fused_all_gather(xs.reshape(-1, xs.shape[-1]), group)
                if g is not None:
                    total = g.view(xs.shape[0] * tp, *xs.shape[1:])
            if total is None:
                total = MemoryBuffer().get("allgather", (xs.shape[0] * tp, *xs.shape[1:]), dtype=xs.dtype, device=xs.device)
                if ctx.async_comm:
                    handle = dist.all_gather_into_tensor(total, xs, group=group, async_op=True)
                else:
                    dist.all_gather_into_tensor(total, xs, group=group)
        else:
            total = saved_in
        go2, _ = _flatten2d(grad_output)
        grad_input = grad_weight = grad_bias = None
        sub_handle = None
        if ctx.needs_input_grad[0]:
            gi_fused = None
            if fused_ok and pre == "all_gather":
                # dgrad GEMM whose epilogue scatters the partial sums to their owners (GEMM -> reduce-scatter)
                gi_fused = ops.tp_fused.fused_matmul_reduce_scatter(go2, weight, group, b_mn=True)
            if gi_fused is not None:
                grad_input = gi_fused.view(grad_output.shape[0] // tp, *grad_output.shape[1:-1], weight.shape[1])
            else:
                gi2 = ops.linear_dgrad(go2, weight)
                gi = gi2.view(*grad_output.shape[:-1], weight.shape[1])
                if tp > 1 and pre == "all_gather":
                    out_gi = torch.empty((gi.shape[0] // tp, *gi.shape[1:]), dtype=gi.dtype, device=gi.device)
                    if ctx.async_comm:
                        sub_handle = dist.reduce_scatter_tensor(out_gi, gi, group=group, async_op=True)
                    else:
                        dist.reduce_scatter_tensor(out_gi, gi, group=group)
                    grad_input = out_gi
                elif tp > 1 and ctx.input_grad_reduce:
                    if ctx.async_comm:
                        sub_handle = dist.all_reduce(gi, group=group, async_op=True)
                    else:
                        dist.all_reduce(gi, group=group)
                    grad_input = gi
                else:
                    grad_input = gi
        if handle is not None:
            handle.wait()
        if weight.requires_grad or ctx.needs_input_grad[1]:
            t2, _ = _flatten2d(total)
            grad_weight = ops.linear_wgrad(go2, t2, weight)
        if ctx.use_bias and ctx.needs_input_grad[2]:
            grad_bias = go2.sum(dim=0)
        if sub_handle is not None:
            sub_handle.wait()
        return grad_input, grad_weight, grad_bias, None, None, None, None, None, None


def column_linear(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    group: Optional[dist.ProcessGroup],
    tp_mode: TensorParallelLinearMode,
    async_communication: bool,
    tp_recompute_allgather: bool = True,
) -> torch.Tensor:
    """Output features are sharded.  ALL_REDUCE: input replicated, its gradient all-reduced.
    REDUCE_SCATTER: input sharded on dim 0, gathered before the GEMM, its gradient reduce-scattered."""
    if tp_mode is TensorParallelLinearMode.ALL_REDUCE:
        return _TPLinear.apply(input, weight, bias, group, "none", "none", True, async_communication, False)
    if tp_mode is TensorParallelLinearMode.REDUCE_SCATTER:
        return _TPLinear.apply(input, weight, bias, group, "all_gather", "none", False, async_communication, tp_recompute_allgather)
    raise ValueError(f"Got unexpected mode: {tp_mode}.")


def row_linear(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    group: Optional[dist.ProcessGroup],
    tp_mode: TensorParallelLinearMode,
    async_communication: bool,
) -> torch.Tensor:
    """Input features are sharded; partial outputs are summed over the group (all-reduce) or summed and
    scattered on dim 0 (reduce-scatter).  The bias (held by every rank, zero except on rank 0's copy in the
    reference) is added after the reduction here, so it is applied exactly once."""
    tp = group.size() if group is not None else 1
    if tp_mode is TensorParallelLinearMode.ALL_REDUCE:
        out = _TPLinear.apply(input, weight, None, group, "none", "all_reduce", False, async_communication, False)
    elif tp_mode is TensorParallelLinearMode.REDUCE_SCATTER:
        if async_communication and input.is_cuda and tp > 1:
            out = ops.tp_fused.MatmulReduceScatter.apply(input, weight, group)
        else:
            out = _TPLinear.apply(input, weight, None, group, "none", "reduce_scatter", False, async_communication, False)
    else:
        raise ValueError(f"Got unexpected mode: {tp_mode}.")
    if bias is not None:
        out = out + bias
    return out


# ----------------------------------------------------------------------------- vocab-parallel cross entropy
class _ShardedCrossEntropy(torch.autograd.Function):
    """Cross entropy over logits whose last dim is sharded across ``group``.

    Three small reductions over the group (max, target logit, sum-exp) like the reference
    (reference functional.py:31-113), but computed by a fused online-softmax kernel per shard on GPU and with the
    softmax *not* materialised: backward recomputes ``exp(logit - logZ)`` from the saved logits and log-partition.
    ``z_loss_coef`` > 0 adds ``coef * logZ^2`` per token (returned separately) with gradient ``2*coef*logZ*softmax``.
    """

    @staticmethod
    def forward(ctx, sharded_logits, target, group, z_loss_coef: float):
        tp = group.size() if group is not None else 1
        rank = dist.get_rank(group) if tp > 1 else 0
        vshard = sharded_logits.shape[-1]
        lead = sharded_logits.shape[:-1]
        logits2 = sharded_logits.reshape(-1, vshard)
        tgt = target.reshape(-1)
        vocab_start = rank * vshard
        local_max, local_sumexp, local_tgt = ops.ce_partials(logits2, tgt, vocab_start)
        fused = None
        if tp > 1 and logits2.is_cuda and ops.tp_fused.ENABLED:
            fused = ops.tp_fused.get_context(group)
        if fused is not None:
            logz, loss = fused.ce_combine(local_max, local_sumexp, local_tgt)  # tp reduction by peer loads inside the kernel
            ctx.save_for_backward(logits2, tgt, logz)
            ctx.vocab_start, ctx.lead, ctx.z = vocab_start, lead, z_loss_coef
            if z_loss_coef > 0:
                return loss.view(lead), (z_loss_coef * logz.square()).view(lead)
            return loss.view(lead), None
        if tp > 1:
            gmax = local_max.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            packed = torch.stack([local_sumexp * torch.exp(local_max - gmax), local_tgt])
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
            sumexp, tgt_logit = packed[0], packed[1]
        else:
            gmax, sumexp, tgt_logit = local_max, local_sumexp, local_tgt
        logz = gmax + torch.log(sumexp)
        loss = logz - tgt_logit
        ctx.save_for_backward(logits2, tgt, logz)
        ctx.vocab_start, ctx.lead, ctx.z = vocab_start, lead, z_loss_coef
        if z_loss_coef > 0:
            z = z_loss_coef * logz.square()
            return loss.view(lead), z.view(lead)
        return loss.view(lead), None

    @staticmethod
    def backward(ctx, grad_loss, grad_z):
        logits2, tgt, logz = ctx.saved_tensors
        g = grad_loss.reshape(-1).contiguous().float()
        gz = None
        if ctx.z > 0:
            gz_in = grad_z.reshape(-1).float() if grad_z is not None else torch.zeros_like(g)
            gz = 2.0 * ctx.z * logz * gz_in
        grad_logits = ops.ce_backward(logits2, tgt, logz, g, gz, ctx.vocab_start)
        return grad_logits.view(*ctx.lead, logits2.shape[-1]), None, None, None


def sharded_cross_entropy(sharded_logits, target, group: Optional[dist.ProcessGroup], dtype: Optional[torch.dtype] = None):
    """Per-token loss in fp32.  ``dtype`` is accepted for signature parity; statistics are always fp32."""
    loss, _ = _ShardedCrossEntropy.apply(sharded_logits, target, group, 0.0)
    return loss


def sharded_cross_entropy_with_z_loss(sharded_logits, target, group, dtype=None, z_loss_coef: float = 1e-4):
    """Returns (per-token CE, per-token z-loss term)."""
    return _ShardedCrossEntropy.apply(sharded_logits, target, group, float(z_loss_coef))


__all__ = [
    "column_linear",
    "row_linear",
    "sharded_cross_entropy",
    "sharded_cross_entropy_with_z_loss",
    "differentiable_identity",
    "differentiable_all_reduce_sum",
]
