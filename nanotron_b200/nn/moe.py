"""Mixture-of-experts layer with expert parallelism (capability parity and beyond: reference src/nanotron/nn/moe.py:26-213
has the router / grouped MLP / shared expert but no expert-parallel communication and no auxiliary loss).

Routing: fp32 router logits -> softmax -> top-k (probabilities are the softmax values of the chosen experts, not
renormalised, like the reference).  Auxiliary load-balance loss per layer (Switch-Transformer form):
``aux = E * sum_e f_e * P_e`` with ``f_e`` the fraction of (token, slot) assignments routed to expert e and ``P_e`` the
mean router probability of expert e; it is returned to the model, which adds ``router_aux_loss_coef * sum_layers aux``.

Expert parallelism: the E experts are split over ``ep_pg`` (consecutive blocks).  Tokens are permuted by expert,
exchanged with a variable-size all-to-all (counts first), processed by the local experts as a grouped GEMM with
device-side offsets, sent back, and combined weighted by the router probabilities.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200.models.base import ignore_init_on_device_and_dtype
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.parallel.sharded_parameters import SplitConfig, create_sharded_parameter_from_config


FUSED_EXPERTS = True  # tests switch this off to compare the kernels with the PyTorch dispatch / grouped-GEMM path


class Router(nn.Module):
    """fp32 linear scorer h -> E; returns (top-k probs [T,k], top-k expert ids int32 [T,k], full probs [T,E])."""

    @ignore_init_on_device_and_dtype
    def __init__(self, config, parallel_config, layer_idx: int):
        super().__init__()
        self.config = config
        self.num_experts = config.moe_config.num_experts
        self.num_experts_per_token = config.moe_config.top_k
        self.weight = nn.Parameter(torch.randn(self.num_experts, config.hidden_size, dtype=torch.float32))

    def gating(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x.to(torch.float32), self.weight.to(torch.float32), bias=None)

    def routing(self, logits: torch.Tensor):
        probs = F.softmax(logits, dim=-1, dtype=torch.float32)
        top_p, top_i = torch.topk(probs, k=self.num_experts_per_token, dim=-1)
        return top_p, top_i.to(torch.int32), probs

    def forward(self, x: torch.Tensor, return_counts: bool = False):
        """With ``return_counts`` a fourth value is returned: int32 [E] assignments per expert (computed by the fused
        kernel on CUDA, by ``bincount`` otherwise)."""
        if x.is_cuda:
            from nanotron_b200 import ops
            from nanotron_b200.ops import native

            if ops.get_mode() != "torch" and native.moe_router_supported(x, self.weight, self.num_experts_per_token):
                top_p, top_i, probs, counts = _FusedRouter.apply(x, self.weight, self.num_experts_per_token)
                return (top_p, top_i, probs, counts) if return_counts else (top_p, top_i, probs)
        top_p, top_i, probs = self.routing(self.gating(x))
        if return_counts:
            return top_p, top_i, probs, torch.bincount(top_i.reshape(-1).long(), minlength=self.num_experts).to(torch.int32)
        return top_p, top_i, probs


class _FusedRouter(torch.autograd.Function):
    """Router forward as one kernel (fp32 logits, softmax, top-k, histogram); backward is the softmax Jacobian applied to
    the gradients that reach the selected probabilities and the full distribution (auxiliary loss)."""

    @staticmethod
    def forward(ctx, x, weight, k):
        from nanotron_b200.ops import native

        top_p, top_i, probs, counts = native.moe_router_fwd(x, weight, k)
        ctx.save_for_backward(x, weight, probs, top_i)
        ctx.mark_non_differentiable(top_i, counts)
        return top_p, top_i, probs, counts

    @staticmethod
    def backward(ctx, d_top_p, _d_top_i, d_probs, _d_counts):
        x, weight, probs, top_i = ctx.saved_tensors
        d = d_probs.clone() if d_probs is not None else torch.zeros_like(probs)
        if d_top_p is not None:
            d.scatter_add_(1, top_i.long(), d_top_p.float())
        dlogits = probs * (d - (d * probs).sum(-1, keepdim=True))
        dw = dlogits.t() @ x.float()
        dx = (dlogits @ weight).to(x.dtype)
        return dx, dw, None


def grouped_mlp_reference(x_sorted, counts, w_gate_up, w_down):
    """Oracle grouped MLP: rows of ``x_sorted`` are grouped by expert with ``counts`` rows each."""
    from nanotron_b200 import ops

    outs = []
    start = 0
    for e, n in enumerate(counts.tolist()):
        xe = x_sorted[start : start + n]
        h = xe @ w_gate_up[e]
        outs.append(ops.swiglu(h) @ w_down[e])
        start += n
    return torch.cat(outs, dim=0) if outs else x_sorted.new_zeros((0, w_down.shape[-1]))


class GroupedMLP(nn.Module):
    """Local experts' weights: ``merged_gate_up_proj [E_local, h, 2I]`` and ``merged_down_proj [E_local, I, h]``."""

    def __init__(self, config, parallel_config, ep_pg: Optional[dist.ProcessGroup] = None):
        super().__init__()
        moe = config.moe_config
        ep = ep_pg.size() if ep_pg is not None else 1
        assert moe.num_experts % ep == 0, f"num_experts ({moe.num_experts}) must be divisible by expert_parallel_size ({ep})"
        self.num_local_experts = moe.num_experts // ep
        self.ep_pg = ep_pg
        h, inter = config.hidden_size, moe.moe_intermediate_size
        self.merged_gate_up_proj = nn.Parameter(torch.empty(self.num_local_experts, h, 2 * inter))
        self.merged_down_proj = nn.Parameter(torch.empty(self.num_local_experts, inter, h))
        if ep > 1:
            self.merged_gate_up_proj = create_sharded_parameter_from_config(self.merged_gate_up_proj, pg=ep_pg, split_config=SplitConfig(split_dim=0))
            self.merged_down_proj = create_sharded_parameter_from_config(self.merged_down_proj, pg=ep_pg, split_config=SplitConfig(split_dim=0))

    def forward(self, x_sorted: torch.Tensor, counts: torch.Tensor) -> Dict[str, torch.Tensor]:
        """x_sorted: [N, h] rows grouped by local expert; counts: int64 [E_local] on the same device."""
        from nanotron_b200 import ops

        if x_sorted.is_cuda and ops.get_mode() != "torch":
            from nanotron_b200.ops import grouped

            out = grouped.grouped_mlp(x_sorted, counts, self.merged_gate_up_proj, self.merged_down_proj)
        else:
            out = grouped_mlp_reference(x_sorted, counts, self.merged_gate_up_proj, self.merged_down_proj)
        return {"hidden_states": out}


class _AllToAllVariable(torch.autograd.Function):
    """Variable-size all-to-all on dim 0 with known split sizes; backward swaps the split lists."""

    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.group, ctx.send_splits, ctx.recv_splits = group, send_splits, recv_splits
        out = x.new_empty((sum(recv_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send_splits), *g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send_splits, input_split_sizes=ctx.recv_splits, group=ctx.group)
        return out, None, None, None


class Qwen2MoELayer(nn.Module):
    def __init__(self, config, parallel_config, tp_pg: dist.ProcessGroup, ep_pg: Optional[dist.ProcessGroup] = None, layer_idx: int = 0):
        super().__init__()
        moe = config.moe_config
        self.hidden_size = config.hidden_size
        self.num_experts = moe.num_experts
        self.top_k = moe.top_k
        self.ep_pg = ep_pg if ep_pg is not None and ep_pg.size() > 1 else None
        self.ep = self.ep_pg.size() if self.ep_pg is not None else 1
        self.num_local_experts = self.num_experts // self.ep
        self.layer_idx = layer_idx
        self.router = Router(config, parallel_config, layer_idx)
        self.experts = GroupedMLP(config, parallel_config, ep_pg=self.ep_pg)
        self.enable_shared_expert = moe.enable_shared_expert
        if self.enable_shared_expert:
            from nanotron_b200.models.qwen import Qwen2MLP

            self.shared_expert = Qwen2MLP(config, parallel_config, tp_pg, intermediate_size=moe.shared_expert_intermediate_size)
            self.shared_expert_gate = nn.Linear(config.hidden_size, 1, bias=False)
        self.recompute_layer = parallel_config.recompute_layer if parallel_config is not None else False

    def _dispatch_compute_combine(self, x, top_p, top_i):
        T, h = x.shape
        k = self.top_k
        flat_e = top_i.reshape(-1).long()  # [T*k], expert of each (token, slot)
        order = torch.argsort(flat_e, stable=True)
        token_of = order // k
        x_sorted = x.index_select(0, token_of)  # rows grouped by global expert id
        counts = torch.bincount(flat_e, minlength=self.num_experts)
        if self.ep == 1:
            y_sorted = self.experts(x_sorted, counts)["hidden_states"]
        else:
            # counts exchange: how many rows each peer sends me, per local expert
            send_counts = counts.view(self.ep, self.num_local_experts)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts.view(-1), send_counts.reshape(-1).contiguous(), group=self.ep_pg)
            send_splits = send_counts.sum(1).tolist()
            recv_splits = recv_counts.sum(1).tolist()
            recv = _AllToAllVariable.apply(x_sorted, send_splits, recv_splits, self.ep_pg)
            # received rows are grouped (peer, local expert); regroup to (local expert, peer)
            seg = recv_counts.reshape(-1)  # [ep*E_local] sizes in arrival order
            seg_expert = torch.arange(self.num_local_experts, device=x.device).repeat(self.ep)
            row_expert = torch.repeat_interleave(seg_expert, seg, output_size=recv.shape[0])
            perm = torch.argsort(row_expert, stable=True)
            local_counts = recv_counts.sum(0)
            y_local = self.experts(recv.index_select(0, perm), local_counts)["hidden_states"]
            y_arrival = torch.empty_like(y_local).index_copy(0, perm, y_local)
            y_sorted = _AllToAllVariable.apply(y_arrival, recv_splits, send_splits, self.ep_pg)
        w = top_p.reshape(-1).index_select(0, order).to(y_sorted.dtype)
        out = torch.zeros((T, h), dtype=y_sorted.dtype, device=x.device)
        out.index_add_(0, token_of, y_sorted * w.unsqueeze(-1))
        return out, counts

    def _fused_path(self, x: torch.Tensor) -> bool:
        if not x.is_cuda:
            return False
        from nanotron_b200 import ops
        from nanotron_b200.ops import moe_fused

        if ops.get_mode() == "torch" or not FUSED_EXPERTS:
            return False
        return moe_fused.supported(x, self.experts.merged_gate_up_proj, self.experts.merged_down_proj, self.num_experts, self.top_k, self.ep_pg)

    def _core_forward(self, hidden_states: torch.Tensor):
        x = hidden_states
        top_p, top_i, probs, counts = self.router(x, return_counts=True)
        if self._fused_path(x):
            from nanotron_b200.ops import moe_fused

            out = moe_fused.fused_moe_experts(x, top_p, top_i, counts, self.experts.merged_gate_up_proj, self.experts.merged_down_proj, self.ep_pg)
        else:
            out, counts = self._dispatch_compute_combine(x, top_p, top_i)
        # load-balance auxiliary loss: E * sum_e f_e * P_e
        f = counts.to(torch.float32) / max(1, top_i.numel())
        P = probs.mean(dim=0)
        aux = self.num_experts * torch.sum(f.detach() * P)
        if self.enable_shared_expert:
            shared = self.shared_expert(hidden_states=x)["hidden_states"]
            gate = torch.sigmoid(self.shared_expert_gate(x))
            out = out + shared * gate
        return out, aux

    def forward(self, hidden_states: torch.Tensor):
        if self.recompute_layer and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            out, aux = checkpoint(self._core_forward, hidden_states, use_reentrant=False)
        else:
            out, aux = self._core_forward(hidden_states)
        return {"hidden_states": out, "aux_loss": aux}
