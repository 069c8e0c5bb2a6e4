"""Starcoder2 / GPT-style decoder: LayerNorm, GELU MLP with biases, dropout, multi-query or grouped-query attention,
optional sliding window with selected global layers (parity: reference src/nanotron/models/starcoder2.py:61-1682).

Module tree and parameter names follow the reference: ``model.token_embeddings.pp_block.token_embedding``,
``model.decoder.{i}.pp_block.{ln_1, attn.qkv.q, attn.qkv.kv, attn.o | attn.query_key_value, attn.dense, ln_2, ff.c_fc, ff.c_proj}``,
``model.final_layer_norm.pp_block``, ``model.lm_head.pp_block``.

Multi-query attention under tensor parallelism: q heads are column-sharded, the single kv head is replicated and
tied over tp with a SUM reduction of its gradients.  The input is brought to full/replicated form once
(all-gather under sequence parallelism, identity otherwise) and feeds both projections, so there is one collective
per direction where the reference needed a dedicated autograd function
(reference starcoder2.py:313-502).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import nn
from torch.nn import functional as F
from torch.utils.checkpoint import checkpoint

from nanotron_b200 import distributed as dist
from nanotron_b200 import ops
from nanotron_b200.config import ParallelismArgs, Starcoder2Config
from nanotron_b200.generation.generate_store import AttachableStore
from nanotron_b200.models.base import NanotronModel
from nanotron_b200.models.qwen import Loss, Qwen2ForTraining, get_flops
from nanotron_b200.nn.activations import ACT2FN
from nanotron_b200.nn.attention import regular_cu_seqlens
from nanotron_b200.nn.layer_norm import TritonLayerNorm
from nanotron_b200.nn.rotary import RotaryEmbedding
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock, TensorPointer
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
from nanotron_b200.parallel.sharded_parameters import SplitConfig, mark_all_parameters_in_module_as_sharded
from nanotron_b200.parallel.tensor_parallel.distributed_differentiable_primitives import differentiable_all_gather, differentiable_identity
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.tensor_parallel.nn import TensorParallelColumnLinear, TensorParallelEmbedding, TensorParallelRowLinear
from nanotron_b200.parallel.tied_parameters import tie_parameters
from nanotron_b200.random import RandomStates, branch_random_state


class MLP(nn.Module):
    def __init__(self, config: Starcoder2Config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup):
        super().__init__()
        tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        async_comm = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        d_ff = config.n_inner if config.n_inner is not None else 4 * config.hidden_size
        self.c_fc = TensorParallelColumnLinear(config.hidden_size, d_ff, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm)
        self.act = ACT2FN[config.activation_function]
        self.c_proj = TensorParallelRowLinear(d_ff, config.hidden_size, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm and tp_mode is TensorParallelLinearMode.REDUCE_SCATTER)

    def forward(self, hidden_states):
        return {"hidden_states": self.c_proj(self.act(self.c_fc(hidden_states)))}


class _Linear(nn.Module):
    """Holds ``weight`` / ``bias`` only (the enclosing module does the matmul)."""

    def __init__(self, in_features: int, out_features: int, bias: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            nn.init.zeros_(self.bias)


class _LocalLinear(torch.autograd.Function):
    """y = x W^T (+ b) with the three products on ``ops.linear_*`` (the in-tree GEMM kernels on CUDA, fp32 main-grad accumulation)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.use_bias = bias is not None
        return ops.linear_forward(x.reshape(-1, x.shape[-1]), weight, bias).view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, go):
        x, weight = ctx.saved_tensors
        go2 = go.reshape(-1, go.shape[-1]).contiguous()
        gx = ops.linear_dgrad(go2, weight).view(x.shape) if ctx.needs_input_grad[0] else None
        gw = ops.linear_wgrad(go2, x.reshape(-1, x.shape[-1]), weight)
        gb = go2.sum(0) if ctx.use_bias else None
        return gx, gw, gb


def _linear(x, weight, bias):
    return _LocalLinear.apply(x, weight, bias)


class MQAColumnLinears(nn.Module):
    def __init__(self, in_features: int, q_out_features: int, kv_out_features: int, pg: dist.ProcessGroup, mode: TensorParallelLinearMode, bias=True, async_communication: bool = False):
        super().__init__()
        self.pg, self.mode = pg, mode
        self.world_size = pg.size()
        assert q_out_features % self.world_size == 0
        self.q_out_features = q_out_features // self.world_size
        self.kv_out_features = kv_out_features
        self.q = _Linear(in_features, self.q_out_features, bias)
        self.kv = _Linear(in_features, kv_out_features, bias)
        mark_all_parameters_in_module_as_sharded(self.q, pg=pg, split_config=SplitConfig(split_dim=0))

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.mode is TensorParallelLinearMode.REDUCE_SCATTER:
            x = differentiable_all_gather(x, group=self.pg)
        else:
            x = differentiable_identity(x, group=self.pg)
        return _linear(x, self.q.weight, self.q.bias), _linear(x, self.kv.weight, self.kv.bias)


class _AttentionBase(nn.Module, AttachableStore):
    def _init_common(self, config: Starcoder2Config, tp_pg, layer_idx: int):
        self.config = config
        self.tp_pg = tp_pg
        self.d_qk = config.hidden_size // config.num_attention_heads
        self.layer_idx = layer_idx
        self.attn_pdrop = config.attn_pdrop
        self.window = None if (config.sliding_window_size is None or layer_idx in (config.global_attn_layers or [])) else config.sliding_window_size
        if config.use_rotary_embeddings:
            self.rotary = RotaryEmbedding(dim=self.d_qk, max_seq_len=config.max_position_embeddings, base=float(config.rope_theta), interleaved=True)
        else:
            self.rotary = None

    def _attend(self, q, k, v, sequence_mask):
        """q [T,Hq,D], k/v [T,Hkv,D]; rows of ``sequence_mask`` [b,s] are whole sequences.  Training batches are padded on the right
        (causal masking hides that from the real tokens); in evaluation mode left padding is kept out of the attention, and with a
        key/value store attached (generation) only the new positions are computed against the cached keys and values
        (reference: the flash_attn_with_kvcache paths, src/nanotron/models/starcoder2.py:832,1077)."""
        b, s = sequence_mask.shape
        scale = (1.0 / math.sqrt(self.d_qk)) if self.config.scale_attn_weights else 1.0
        store = self.get_local_store()
        if store is not None:
            return self._attend_cached(q, k, v, sequence_mask, store, scale)
        if self.rotary is not None:
            pos = (sequence_mask.long().cumsum(-1) - 1).clamp_(min=0).reshape(-1)
            q, k = self.rotary(q, k, pos)
        cu = None
        if not self.training:
            from nanotron_b200.models.llama import padding_cu_seqlens

            cu = padding_cu_seqlens(sequence_mask)
        if cu is None:
            cu = regular_cu_seqlens(b, s, q.device)
        return ops.flash_attn_varlen(q, k, v, cu, cu, s, s, causal=True, softmax_scale=scale, window=self.window)

    def _attend_cached(self, q, k, v, sequence_mask, store, scale):
        from nanotron_b200.nn.attention import cached_attention

        b, qlen = sequence_mask.shape
        Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
        past_len = store.get("past_len", torch.zeros(b, dtype=torch.long, device=q.device))
        if self.rotary is not None:
            pos = (past_len.unsqueeze(1) + (sequence_mask.long().cumsum(-1) - 1).clamp_(min=0)).reshape(-1)
            q, k = self.rotary(q, k, pos)
        kb, vb = k.reshape(b, qlen, Hkv, D), v.reshape(b, qlen, Hkv, D)
        if "key" in store:
            k_all, v_all = torch.cat([store["key"], kb], dim=1), torch.cat([store["value"], vb], dim=1)
            m_all = torch.cat([store["mask"], sequence_mask.bool()], dim=1)
        else:
            k_all, v_all, m_all = kb, vb, sequence_mask.bool()
        store.update({"key": k_all, "value": v_all, "mask": m_all, "past_len": past_len + sequence_mask.long().sum(-1)})
        out = cached_attention(q.reshape(b, qlen, Hq, D), k_all, v_all, sequence_mask.bool(), m_all, softmax_scale=scale, sliding_window=self.window)
        return out.reshape(b * qlen, Hq, D)


class CausalSelfMQA(_AttentionBase):
    def __init__(self, config: Starcoder2Config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, layer_idx: int):
        super().__init__()
        self._init_common(config, tp_pg, layer_idx)
        tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        async_comm = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        assert config.num_attention_heads % tp_pg.size() == 0
        self.n_local_heads = config.num_attention_heads // tp_pg.size()
        self.qkv = MQAColumnLinears(config.hidden_size, config.num_attention_heads * self.d_qk, 2 * self.d_qk, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm)
        self.o = TensorParallelRowLinear(config.num_attention_heads * self.d_qk, config.hidden_size, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm and tp_mode is TensorParallelLinearMode.REDUCE_SCATTER)

    def forward(self, hidden_states, sequence_mask):
        q, kv = self.qkv(hidden_states)
        T = q.shape[0]
        q = q.view(T, self.n_local_heads, self.d_qk)
        k, v = kv.view(T, 2, 1, self.d_qk).unbind(dim=1)
        out = self._attend(q, k.contiguous(), v.contiguous(), sequence_mask)
        return {"hidden_states": self.o(out.reshape(T, self.n_local_heads * self.d_qk)), "sequence_mask": sequence_mask}


class CausalSelfGQA(_AttentionBase):
    def __init__(self, config: Starcoder2Config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, layer_idx: int):
        super().__init__()
        self._init_common(config, tp_pg, layer_idx)
        tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        async_comm = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        tp = tp_pg.size()
        assert config.num_attention_heads % tp == 0 and config.num_kv_heads % tp == 0
        self.n_local_heads = config.num_attention_heads // tp
        self.n_local_kv = config.num_kv_heads // tp
        q_size, kv_size = config.num_attention_heads * self.d_qk, config.num_kv_heads * self.d_qk
        self.query_key_value = TensorParallelColumnLinear(config.hidden_size, q_size + 2 * kv_size, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm, contiguous_chunks=(q_size, kv_size, kv_size))
        self.dense = TensorParallelRowLinear(q_size, config.hidden_size, pg=tp_pg, mode=tp_mode, bias=True, async_communication=async_comm and tp_mode is TensorParallelLinearMode.REDUCE_SCATTER)

    def forward(self, hidden_states, sequence_mask):
        qkv = self.query_key_value(hidden_states)
        T = qkv.shape[0]
        lq, lkv = self.n_local_heads * self.d_qk, self.n_local_kv * self.d_qk
        q = qkv[:, :lq].view(T, self.n_local_heads, self.d_qk)
        k = qkv[:, lq : lq + lkv].view(T, self.n_local_kv, self.d_qk)
        v = qkv[:, lq + lkv :].view(T, self.n_local_kv, self.d_qk)
        out = self._attend(q, k, v, sequence_mask)
        return {"hidden_states": self.dense(out.reshape(T, lq)), "sequence_mask": sequence_mask}


def dropout_add(x, residual, prob, training):
    return residual + F.dropout(x, p=prob, training=training)


class GPTBlock(nn.Module):
    def __init__(self, config: Starcoder2Config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, random_states: RandomStates, layer_idx: int):
        super().__init__()
        self.ln_1 = TritonLayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        if config.multi_query:
            self.attn = CausalSelfMQA(config, parallel_config, tp_pg, layer_idx)
        elif config.grouped_query:
            self.attn = CausalSelfGQA(config, parallel_config, tp_pg, layer_idx)
        else:
            raise ValueError("Either `multi_query` or `grouped_query` must be True")
        self.attn_dropout = config.attn_pdrop
        self.ln_2 = TritonLayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.ff = MLP(config, parallel_config, tp_pg)
        self.ff_dropout = config.resid_pdrop
        self.random_states = random_states
        self.tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        self.recompute_layer = parallel_config.recompute_layer if parallel_config is not None else False

    def _core(self, hidden_states, sequence_mask):
        residual = hidden_states
        h = self.ln_1(hidden_states)
        h = self.attn(hidden_states=h, sequence_mask=sequence_mask)["hidden_states"]
        # replicated activations must see the same dropout mask on every tp rank
        with branch_random_state(self.random_states, "tp_synced", enabled=self.tp_mode is TensorParallelLinearMode.ALL_REDUCE and self.training and self.attn_dropout > 0):
            h = dropout_add(h, residual, self.attn_dropout, self.training)
        residual = h
        h = self.ln_2(h)
        h = self.ff(hidden_states=h)["hidden_states"]
        with branch_random_state(self.random_states, "tp_synced", enabled=self.tp_mode is TensorParallelLinearMode.ALL_REDUCE and self.training and self.ff_dropout > 0):
            h = dropout_add(h, residual, self.ff_dropout, self.training)
        return h

    def forward(self, hidden_states, sequence_mask):
        if self.recompute_layer and not isinstance(hidden_states, TensorPointer) and torch.is_grad_enabled():
            h = checkpoint(self._core, hidden_states, sequence_mask, use_reentrant=False)
        else:
            h = self._core(hidden_states, sequence_mask)
        return {"hidden_states": h, "sequence_mask": sequence_mask}


class Embedding(nn.Module, AttachableStore):
    def __init__(self, tp_pg: dist.ProcessGroup, config: Starcoder2Config, parallel_config: Optional[ParallelismArgs]):
        super().__init__()
        self.token_embedding = TensorParallelEmbedding(num_embeddings=config.vocab_size, embedding_dim=config.hidden_size, pg=tp_pg, mode=parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE)
        self.pg = tp_pg

    def forward(self, input_ids: torch.Tensor, input_mask: torch.Tensor):
        return {"input_embeds": self.token_embedding(input_ids.reshape(-1))}


class _Dropout(nn.Module):
    def __init__(self, p: float):
        super().__init__()
        self.p = p

    def forward(self, input):
        return {"hidden_states": F.dropout(input, p=self.p, training=self.training)}


class GPTModel(nn.Module):
    def __init__(self, config: Starcoder2Config, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs], random_states: RandomStates):
        super().__init__()
        self.p2p = P2P(parallel_context.pp_pg, device=parallel_context.device)
        self.config, self.parallel_context, self.parallel_config = config, parallel_context, parallel_config
        self.random_states = random_states
        self.tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        self.token_embeddings = PipelineBlock(p2p=self.p2p, module_builder=Embedding, module_kwargs={"tp_pg": parallel_context.tp_pg, "config": config, "parallel_config": parallel_config}, module_input_keys={"input_ids", "input_mask"}, module_output_keys={"input_embeds"})
        self.embeds_dropout = PipelineBlock(p2p=self.p2p, module_builder=_Dropout, module_kwargs={"p": config.embd_pdrop}, module_input_keys={"input"}, module_output_keys={"hidden_states"})
        self.decoder = nn.ModuleList(
            [
                PipelineBlock(p2p=self.p2p, module_builder=GPTBlock, module_kwargs={"config": config, "parallel_config": parallel_config, "tp_pg": parallel_context.tp_pg, "random_states": random_states, "layer_idx": i}, module_input_keys={"hidden_states", "sequence_mask"}, module_output_keys={"hidden_states", "sequence_mask"})
                for i in range(config.num_hidden_layers)
            ]
        )
        self.final_layer_norm = PipelineBlock(p2p=self.p2p, module_builder=TritonLayerNorm, module_kwargs={"normalized_shape": config.hidden_size, "eps": config.layer_norm_epsilon}, module_input_keys={"input"}, module_output_keys={"hidden_states"})
        self.lm_head = PipelineBlock(
            p2p=self.p2p, module_builder=TensorParallelColumnLinear,
            module_kwargs={"in_features": config.hidden_size, "out_features": config.vocab_size, "pg": parallel_context.tp_pg, "bias": False, "mode": self.tp_mode, "async_communication": parallel_config.tp_linear_async_communication if parallel_config is not None else False},
            module_input_keys={"x"}, module_output_keys={"logits"},
        )

    def forward(self, input_ids, input_mask):
        h = self.token_embeddings(input_ids=input_ids, input_mask=input_mask)["input_embeds"]
        with branch_random_state(self.random_states, "tp_synced", enabled=self.tp_mode is TensorParallelLinearMode.ALL_REDUCE and self.training and self.config.embd_pdrop > 0):
            h = self.embeds_dropout(input=h)["hidden_states"]
        state = {"hidden_states": h, "sequence_mask": input_mask}
        for layer in self.decoder:
            state = layer(**state)
        h = self.final_layer_norm(input=state["hidden_states"])["hidden_states"]
        return self.lm_head(x=h)["logits"]

    def get_block_compute_costs(self):
        c = self.config
        d_ff = c.n_inner if c.n_inner is not None else 4 * c.hidden_size
        d_qkv = c.hidden_size // c.num_attention_heads
        kv = 1 if c.multi_query else c.num_kv_heads
        return {
            GPTBlock: 2 * c.num_attention_heads * d_qkv * c.hidden_size + 2 * kv * d_qkv * c.hidden_size + 2 * d_ff * c.hidden_size,
            TensorParallelColumnLinear: c.vocab_size * c.hidden_size,
        }

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        world = self.parallel_context.world_pg.size()
        c = self.config
        d_ff = c.n_inner if c.n_inner is not None else 4 * c.hidden_size
        kv = 1 if c.multi_query else c.num_kv_heads
        # 2-matrix MLP: count as a gated MLP of 2/3 the width so the shared formula applies
        model_flops, hardware_flops = get_flops(num_layers=c.num_hidden_layers, hidden_size=c.hidden_size, num_heads=c.num_attention_heads, num_key_value_heads=kv, vocab_size=c.vocab_size, ffn_hidden_size=d_ff * 2 / 3, seq_len=sequence_length, batch_size=global_batch_size)
        return model_flops / (iteration_time_in_sec * world * 1e12), hardware_flops / (iteration_time_in_sec * world * 1e12)


class Starcoder2ForTraining(NanotronModel):
    def __init__(self, config: Starcoder2Config, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs], random_states: Optional[RandomStates] = None):
        super().__init__()
        if random_states is None:
            random_states = RandomStates({})
        self.model = GPTModel(config=config, parallel_context=parallel_context, parallel_config=parallel_config, random_states=random_states)
        self.loss = PipelineBlock(p2p=self.model.p2p, module_builder=Loss, module_kwargs={"tp_pg": parallel_context.tp_pg}, module_input_keys={"sharded_logits", "label_ids", "label_mask"}, module_output_keys={"loss"})
        self.config, self.parallel_config, self.parallel_context = config, parallel_config, parallel_context

    def forward(self, input_ids, input_mask, label_ids, label_mask):
        logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return {"loss": self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask)["loss"]}

    def tie_custom_params(self) -> None:
        """The replicated kv projection of multi-query attention is tied over tp; its gradients are partial on every
        rank (each saw only its own heads) and are summed."""
        for module_name, module in self.named_modules():
            if not isinstance(module, CausalSelfMQA):
                continue
            tp_ranks = dist.get_global_ranks(self.parallel_context.tp_pg)
            for pname, p in list(module.qkv.kv.named_parameters()):
                if p is None:
                    continue
                name = f"{module_name}.qkv.kv.{pname}"
                tie_parameters(root_module=self, ties=[(name, tp_ranks)], parallel_context=self.parallel_context, reduce_op=dist.ReduceOp.SUM)

    @torch.no_grad()
    def init_model_randomly(self, config):
        std = config.model.init_method.std
        sigma = std / math.sqrt(2 * self.config.num_hidden_layers)
        done = set()
        for name, p in sorted(self.named_parameters(), key=lambda x: x[0]):
            full = p.get_tied_info().get_full_name_from_module_id_to_prefix(self.module_id_to_prefix) if p.is_tied else name
            if full in done:
                continue
            done.add(full)
            module_name, _, local = name.rpartition(".")
            module = self.get_submodule(module_name)
            if local == "bias":
                p.zero_()
            elif isinstance(module, (TritonLayerNorm,)):
                p.fill_(1)
            elif isinstance(module, TensorParallelRowLinear):
                nn.init.normal_(p, mean=0.0, std=sigma)
            else:
                nn.init.normal_(p, mean=0.0, std=std)

    def get_embeddings_lm_head_tied_names(self) -> List[str]:
        return ["model.token_embeddings.pp_block.token_embedding.weight", "model.lm_head.pp_block.weight"]

    def get_block_compute_costs(self):
        return self.model.get_block_compute_costs()

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        return self.model.get_flops_per_sec(iteration_time_in_sec, sequence_length, global_batch_size)
