"""Llama decoder-only transformer (parity: reference src/nanotron/models/llama.py:54-1225).

Same module tree and parameter names as the reference.  Inputs are ``input_ids`` / ``input_mask`` [b, s]; the mask
travels between pipeline blocks as ``sequence_mask``.  Internally the activations use the token-flat layout
``[b*s, h]`` shared with the Qwen2 implementation (the reference uses ``[s, b, h]``); with sequence parallelism the
flat token dimension is what gets sharded.  Positions are derived from the mask (``cumsum(mask) - 1``) so right-padded
batches rotate correctly; padded positions are ignored by the loss mask.
"""
from __future__ import annotations

from typing import Dict, Optional, Union

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from nanotron_b200 import distributed as dist
from nanotron_b200.config import LlamaConfig, ParallelismArgs
from nanotron_b200.models import qwen as _q
from nanotron_b200.models.qwen import Loss, LossWithZLoss, get_flops, masked_mean  # noqa: F401
from nanotron_b200.nn.layer_norm import TritonRMSNorm
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock, TensorPointer
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.tensor_parallel.nn import TensorParallelColumnLinear, TensorParallelEmbedding
from nanotron_b200.random import RandomStates


class MLP(_q.Qwen2MLP):
    pass


def padding_cu_seqlens(sequence_mask: torch.Tensor) -> Optional[torch.Tensor]:
    """Document boundaries that keep padding out of the attention of real tokens, for batches padded on the LEFT (generation,
    evaluation): every padding token becomes a document of its own and the real tokens of a row form one document.  Returns None
    for a mask without padding.  Right padding needs nothing (causal masking already hides it from the real tokens), which is why
    training never calls this.  The result is cached on the mask tensor: every layer of a stage asks for the same one."""
    cached = getattr(sequence_mask, "_ntb_padding_cu", False)
    if cached is not False:
        return cached
    m = sequence_mask.bool()
    if bool(m.all()):
        cu = None
    else:
        b, s = m.shape
        prev = torch.cat([torch.zeros(b, 1, dtype=torch.bool, device=m.device), m[:, :-1]], dim=1)
        starts = (~m) | (~prev)  # a padding token, or the first token after padding / of the row
        idx = torch.nonzero(starts.reshape(-1), as_tuple=False).flatten()
        cu = torch.cat([idx, torch.tensor([b * s], device=m.device)]).to(torch.int32)
    try:
        sequence_mask._ntb_padding_cu = cu
    except AttributeError:
        pass
    return cu


class CausalSelfAttention(_q.Qwen2Attention):
    """Adds a KV-cache decode path (used by ``nanotron_b200.generation``) on top of the training path."""

    def forward(self, hidden_states, sequence_mask, cu_seqlens=None):
        from nanotron_b200.generation.generate_store import AttachableStore  # noqa: F401

        store = self.get_local_store() if hasattr(self, "get_local_store") else None
        if store is not None:
            return self._forward_with_cache(hidden_states, sequence_mask, store)
        position_ids = (sequence_mask.long().cumsum(-1) - 1).clamp_(min=0)
        if cu_seqlens is None and not self.training:
            cu_seqlens = padding_cu_seqlens(sequence_mask)
        out = super().forward(hidden_states, position_ids, cu_seqlens)
        return {"hidden_states": out["hidden_states"], "sequence_mask": sequence_mask}

    def _forward_with_cache(self, hidden_states, sequence_mask, store):
        """Decode with cached K/V.  hidden_states: [b*q, h] for q new tokens per row; ``sequence_mask`` [b, q] marks
        which of the new positions are real (left padding allowed on the first call)."""
        from nanotron_b200.ops import reference as ref

        b, qlen = sequence_mask.shape
        qkv = self.qkv_proj(hidden_states)
        T = qkv.shape[0]
        q = qkv[:, : self.local_q_size].view(b, qlen, self.local_heads, self.head_dim)
        k = qkv[:, self.local_q_size : self.local_q_size + self.local_kv_size].view(b, qlen, self.local_kv_heads, self.head_dim)
        v = qkv[:, self.local_q_size + self.local_kv_size :].view(b, qlen, self.local_kv_heads, self.head_dim)
        past_len = store.get("past_len", torch.zeros(b, dtype=torch.long, device=hidden_states.device))
        pos = past_len.unsqueeze(1) + (sequence_mask.long().cumsum(-1) - 1).clamp_(min=0)
        if self.use_rope:
            cos, sin = self.rotary_emb.get_cos_sin(pos.reshape(-1), max_position=int(pos.max().item()) + 1)
            q = ref.rope_apply(q.reshape(T, self.local_heads, self.head_dim), cos, sin, self.rotary_emb.interleaved).view_as(q)
            k = ref.rope_apply(k.reshape(T, self.local_kv_heads, self.head_dim), cos, sin, self.rotary_emb.interleaved).view_as(k)
        if "key" in store:
            k_all = torch.cat([store["key"], k], dim=1)
            v_all = torch.cat([store["value"], v], dim=1)
            m_all = torch.cat([store["mask"], sequence_mask.bool()], dim=1)
        else:
            k_all, v_all, m_all = k, v, sequence_mask.bool()
        store.update({"key": k_all, "value": v_all, "mask": m_all, "past_len": past_len + sequence_mask.long().sum(-1)})
        from nanotron_b200.nn.attention import cached_attention

        out = cached_attention(q, k_all, v_all, sequence_mask.bool(), m_all, softmax_scale=self.softmax_scale if self.softmax_scale is not None else 1.0 / (self.head_dim**0.5), sliding_window=self.sliding_window_size)
        out = out.reshape(T, self.local_q_size).to(hidden_states.dtype)
        return {"hidden_states": self.o_proj(out), "sequence_mask": sequence_mask}


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, cp_pg=None, layer_idx: int = 0, parallel_context=None):
        super().__init__()
        from nanotron_b200.generation.generate_store import attachable

        self.input_layernorm = TritonRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.attn = attachable(CausalSelfAttention)(config, parallel_config, tp_pg, cp_pg, layer_idx)
        self.post_attention_layernorm = TritonRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.mlp = MLP(config, parallel_config, tp_pg)
        self.recompute_layer = parallel_config.recompute_layer if parallel_config is not None else False

    def _core_forward(self, hidden_states, sequence_mask):
        normed, residual = self.input_layernorm(hidden_states, prenorm=True)
        attn_out = self.attn(hidden_states=normed, sequence_mask=sequence_mask)["hidden_states"]
        normed, residual = self.post_attention_layernorm(attn_out, residual=residual)
        hidden_states = self.mlp(hidden_states=normed)["hidden_states"] + residual
        return hidden_states

    def forward(self, hidden_states, sequence_mask):
        if self.recompute_layer and not isinstance(hidden_states, TensorPointer) and torch.is_grad_enabled():
            hidden_states = checkpoint(self._core_forward, hidden_states, sequence_mask, use_reentrant=False)
        else:
            hidden_states = self._core_forward(hidden_states, sequence_mask)
        return {"hidden_states": hidden_states, "sequence_mask": sequence_mask}


class Embedding(nn.Module):
    def __init__(self, tp_pg: dist.ProcessGroup, config: LlamaConfig, parallel_config: Optional[ParallelismArgs]):
        super().__init__()
        self.token_embedding = TensorParallelEmbedding(
            num_embeddings=config.vocab_size, embedding_dim=config.hidden_size, padding_idx=config.pad_token_id, pg=tp_pg,
            mode=parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE,
        )
        self.pg = tp_pg

    def forward(self, input_ids: torch.Tensor, input_mask: torch.Tensor):
        return {"input_embeds": self.token_embedding(input_ids.reshape(-1))}


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs]):
        super().__init__()
        from nanotron_b200.parallel.pipeline_parallel.p2p import P2P

        self.p2p = P2P(parallel_context.pp_pg, device=parallel_context.device)
        self.config = config
        self.parallel_config = parallel_config
        self.parallel_context = parallel_context
        self.tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        tp_linear_async = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        self.token_position_embeddings = PipelineBlock(
            p2p=self.p2p, module_builder=Embedding,
            module_kwargs={"tp_pg": parallel_context.tp_pg, "config": config, "parallel_config": parallel_config},
            module_input_keys={"input_ids", "input_mask"}, module_output_keys={"input_embeds"},
        )
        self.decoder = nn.ModuleList(
            [
                PipelineBlock(
                    p2p=self.p2p, module_builder=LlamaDecoderLayer,
                    module_kwargs={"config": config, "parallel_config": parallel_config, "tp_pg": parallel_context.tp_pg, "cp_pg": parallel_context.cp_pg, "layer_idx": i},
                    module_input_keys={"hidden_states", "sequence_mask"}, module_output_keys={"hidden_states", "sequence_mask"},
                )
                for i in range(config.num_hidden_layers)
            ]
        )
        self.final_layer_norm = PipelineBlock(
            p2p=self.p2p, module_builder=TritonRMSNorm, module_kwargs={"hidden_size": config.hidden_size, "eps": config.rms_norm_eps},
            module_input_keys={"input"}, module_output_keys={"hidden_states"},
        )
        self.lm_head = PipelineBlock(
            p2p=self.p2p, module_builder=TensorParallelColumnLinear,
            module_kwargs={
                "in_features": config.hidden_size, "out_features": config.vocab_size, "pg": parallel_context.tp_pg, "bias": False,
                "mode": self.tp_mode, "async_communication": tp_linear_async,
                "tp_recompute_allgather": parallel_config.tp_recompute_allgather if parallel_config is not None else True,
            },
            module_input_keys={"x"}, module_output_keys={"logits"},
        )

    def forward(self, input_ids, input_mask):
        return self.forward_with_hidden_states(input_ids=input_ids, input_mask=input_mask)[0]

    def forward_with_hidden_states(self, input_ids, input_mask):
        out = self.token_position_embeddings(input_ids=input_ids, input_mask=input_mask)
        state = {"hidden_states": out["input_embeds"], "sequence_mask": input_mask}
        for layer in self.decoder:
            state = layer(**state)
        hidden = self.final_layer_norm(input=state["hidden_states"])["hidden_states"]
        logits = self.lm_head(x=hidden)["logits"]
        return logits, hidden

    def get_block_compute_costs(self):
        c = self.config
        d_qkv = c.hidden_size // c.num_attention_heads
        return {
            LlamaDecoderLayer: 2 * c.num_attention_heads * d_qkv * c.hidden_size + 2 * c.num_key_value_heads * d_qkv * c.hidden_size + 3 * c.intermediate_size * c.hidden_size,
            TensorParallelColumnLinear: c.vocab_size * c.hidden_size,
        }

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        world = self.parallel_context.world_pg.size()
        c = self.config
        model_flops, hardware_flops = get_flops(
            num_layers=c.num_hidden_layers, hidden_size=c.hidden_size, num_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
            vocab_size=c.vocab_size, ffn_hidden_size=c.intermediate_size, seq_len=sequence_length, batch_size=global_batch_size,
        )
        return model_flops / (iteration_time_in_sec * world * 1e12), hardware_flops / (iteration_time_in_sec * world * 1e12)


class LlamaForTraining(_q.Qwen2ForTraining):
    model_class = LlamaModel

    def forward(self, input_ids, input_mask, label_ids, label_mask) -> Dict[str, Union[torch.Tensor, TensorPointer]]:
        sharded_logits = self.model(input_ids=input_ids, input_mask=input_mask)
        return self.loss(sharded_logits=sharded_logits, label_ids=label_ids, label_mask=label_mask)
