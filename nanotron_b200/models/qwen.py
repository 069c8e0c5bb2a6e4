"""Qwen2 decoder-only transformer (dense and MoE), token-flat activation layout ``[b*s, h]``.

Parity: reference src/nanotron/models/qwen.py:37-1092 (module tree and parameter names are the same:
``model.token_position_embeddings.pp_block.token_embedding.weight``,
``model.decoder.{i}.pp_block.{input_layernorm,attn.qkv_proj,attn.o_proj,post_attention_layernorm,mlp.gate_up_proj,mlp.down_proj}``,
``model.final_layer_norm.pp_block.weight``, ``model.lm_head.pp_block.weight``).

Data flow of one decoder layer on CUDA, all in-tree kernels except plain GEMMs:
fused (residual add +) RMSNorm -> qkv GEMM -> in-place RoPE on the q/k views -> flash attention (varlen, GQA, causal)
-> o GEMM -> fused residual-add + RMSNorm -> gate_up GEMM -> SwiGLU -> down GEMM -> residual add.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Union

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from nanotron_b200 import distributed as dist
from nanotron_b200 import ops
from nanotron_b200.config import Config, ParallelismArgs, Qwen2Config
from nanotron_b200.config.models_config import RandomInit, SpectralMupInit
from nanotron_b200.logging import LogMixin, get_logger
from nanotron_b200.models.base import NanotronModel
from nanotron_b200.nn.activations import GLUActivation
from nanotron_b200.nn.attention import ALL_ATTENTION_FUNCTIONS, get_attention_mask, regular_cu_seqlens
from nanotron_b200.nn.layer_norm import LlamaRMSNorm, TritonRMSNorm
from nanotron_b200.nn.rotary import RotaryEmbedding
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock, TensorPointer
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.tensor_parallel.functional import sharded_cross_entropy, sharded_cross_entropy_with_z_loss
from nanotron_b200.parallel.tensor_parallel.nn import (
    TensorParallelColumnLinear,
    TensorParallelEmbedding,
    TensorParallelRowLinear,
)
from nanotron_b200.random import RandomStates
from nanotron_b200.scaling.parametrization import SpectralMupParametrizator, StandardParametrizator

logger = get_logger(__name__)


class Qwen2MLP(nn.Module):
    def __init__(self, config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, intermediate_size: Optional[int] = None, hidden_act: Optional[str] = None):
        super().__init__()
        tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        async_comm = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        recompute_ag = parallel_config.tp_recompute_allgather if parallel_config is not None else True
        inter = intermediate_size if intermediate_size is not None else config.intermediate_size
        self.gate_up_proj = TensorParallelColumnLinear(
            config.hidden_size, 2 * inter, pg=tp_pg, mode=tp_mode, bias=False, async_communication=async_comm,
            contiguous_chunks=(inter, inter), tp_recompute_allgather=recompute_ag,
        )
        self.down_proj = TensorParallelRowLinear(
            inter, config.hidden_size, pg=tp_pg, mode=tp_mode, bias=False,
            async_communication=async_comm and tp_mode is TensorParallelLinearMode.REDUCE_SCATTER,
        )
        self.split_silu_mul = GLUActivation(hidden_act or getattr(config, "hidden_act", "silu"))

    def forward(self, hidden_states):
        merged = self.gate_up_proj(hidden_states)
        return {"hidden_states": self.down_proj(self.split_silu_mul(merged))}


class Qwen2Attention(nn.Module, LogMixin):
    def __init__(self, config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, cp_pg: Optional[dist.ProcessGroup], layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.tp_pg, self.cp_pg = tp_pg, cp_pg
        self.cp_size = cp_pg.size() if cp_pg is not None else 1
        tp = tp_pg.size()
        tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        async_comm = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        recompute_ag = parallel_config.tp_recompute_allgather if parallel_config is not None else True
        self.tp_mode = tp_mode
        self.hidden_size = config.hidden_size
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.n_heads = config.num_attention_heads
        self.n_kv_heads = config.num_key_value_heads
        assert self.n_heads % tp == 0 and self.n_kv_heads % tp == 0, f"heads ({self.n_heads}, kv {self.n_kv_heads}) must be divisible by tp ({tp})"
        self.local_heads = self.n_heads // tp
        self.local_kv_heads = self.n_kv_heads // tp
        self.local_q_size = self.local_heads * self.head_dim
        self.local_kv_size = self.local_kv_heads * self.head_dim
        q_size, kv_size = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.qkv_proj = TensorParallelColumnLinear(
            self.hidden_size, q_size + 2 * kv_size, pg=tp_pg, mode=tp_mode, bias=getattr(config, "attention_bias", False),
            async_communication=async_comm, contiguous_chunks=(q_size, kv_size, kv_size), tp_recompute_allgather=recompute_ag,
        )
        self.o_proj = TensorParallelRowLinear(
            q_size, self.hidden_size, pg=tp_pg, mode=tp_mode, bias=False,
            async_communication=async_comm and tp_mode is TensorParallelLinearMode.REDUCE_SCATTER,
        )
        no_rope = getattr(config, "no_rope_layer", None)
        self.use_rope = not (no_rope is not None and (layer_idx + 1) % no_rope == 0)
        if self.use_rope:
            self.rotary_emb = RotaryEmbedding(
                dim=self.head_dim, max_seq_len=config.max_position_embeddings, base=config.rope_theta,
                interleaved=config.rope_interleaved, seq_len_scaling_factor=getattr(config, "rope_seq_len_interpolation_factor", None),
                rope_scaling=getattr(config, "rope_scaling", None),
            )
        # spectral muP scales attention logits by 1 / head_dim instead of 1 / sqrt(head_dim) (reference models/llama.py:289)
        self.softmax_scale = 1.0 / self.head_dim if getattr(config, "is_using_mup", False) else None
        self.attn_impl = config._attn_implementation or "flash_attention_2"
        if self.cp_size > 1 and self.attn_impl not in ("ring", "llama3_ring_attention", "ring_flash_triton", "ring_fused"):
            self.attn_impl = "llama3_ring_attention"  # the all-gather variant; "ring" passes K / V blocks around instead
        self.attention = ALL_ATTENTION_FUNCTIONS[self.attn_impl]
        self.sliding_window_size = getattr(config, "sliding_window_size", None)
        self.log_attn_probs = getattr(config, "log_attn_probs", False)

    def forward(self, hidden_states: torch.Tensor, position_ids: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None):
        """hidden_states: [T_local, h] (T_local = b*s/tp under sequence parallelism); position_ids: [b, s_local]."""
        qkv = self.qkv_proj(hidden_states)  # [T, local_q + 2*local_kv]
        T = qkv.shape[0]
        log_stats = self.log_attn_probs and self.training and self.cp_size == 1
        if not log_stats and self.cp_size == 1 and self.attn_impl in ("flash_attention_2", "sdpa") and ops.fused_qkv_attention_supported(qkv, self.local_heads, self.local_kv_heads, self.head_dim, self.sliding_window_size):
            b, s = position_ids.shape
            cu = cu_seqlens if cu_seqlens is not None else regular_cu_seqlens(b, s, hidden_states.device)
            if self.use_rope:
                self.rotary_emb._ensure_tables(self.rotary_emb.max_seq_len, qkv.device)
                cos, sin, interleaved = self.rotary_emb.cos_table, self.rotary_emb.sin_table, self.rotary_emb.interleaved
            else:
                cos = sin = None
                interleaved = False
            out = ops.fused_qkv_attention(qkv, cos, sin, position_ids.reshape(-1), self.local_heads, self.local_kv_heads, self.head_dim, cu, s, causal=True, softmax_scale=self.softmax_scale, window=self.sliding_window_size, interleaved=interleaved, use_rope=self.use_rope)
            out = self.o_proj(out.reshape(T, self.local_q_size))
            return {"hidden_states": out, "position_ids": position_ids}
        if not log_stats and self.cp_size == 1 and self.softmax_scale is None and self.attn_impl == "flash_attention_2" and ops.fused_qkv_library_attention_supported(qkv, self.head_dim, self.sliding_window_size, cu_seqlens):
            b, s = position_ids.shape
            if self.use_rope:
                self.rotary_emb._ensure_tables(self.rotary_emb.max_seq_len, qkv.device)
                cos, sin, interleaved = self.rotary_emb.cos_table, self.rotary_emb.sin_table, self.rotary_emb.interleaved
            else:
                cos = sin = None
                interleaved = False
            out = ops.fused_qkv_library_attention(qkv, cos, sin, position_ids.reshape(-1), self.local_heads, self.local_kv_heads, self.head_dim, b, s, interleaved=interleaved, use_rope=self.use_rope)
            out = self.o_proj(out.reshape(T, self.local_q_size))
            return {"hidden_states": out, "position_ids": position_ids}
        q = qkv[:, : self.local_q_size].view(T, self.local_heads, self.head_dim)
        k = qkv[:, self.local_q_size : self.local_q_size + self.local_kv_size].view(T, self.local_kv_heads, self.head_dim)
        v = qkv[:, self.local_q_size + self.local_kv_size :].view(T, self.local_kv_heads, self.head_dim)
        b, s = position_ids.shape
        if self.use_rope:
            q, k = self.rotary_emb(q, k, position_ids.reshape(-1), inplace=False)
        doc_masking = cu_seqlens is not None  # under context parallelism the exchange cuts at the (global) document starts itself
        if cu_seqlens is None:
            cu_seqlens = regular_cu_seqlens(b, s, hidden_states.device)
        max_len = s
        if log_stats:
            # [local heads, tokens] log-sum-exp of the attention scores, collected by the trainer once per logged step
            self.tbi_logger({"attn_probs": ops.attention_lse(q, k, v, cu_seqlens, cu_seqlens, max_len, max_len, causal=True, softmax_scale=self.softmax_scale, window=self.sliding_window_size)})
        out = self.attention(
            q, k, v, cu_seqlens_q=cu_seqlens, cu_seqlens_k=cu_seqlens, max_seqlen_q=max_len, max_seqlen_k=max_len, causal=True,
            softmax_scale=self.softmax_scale, sliding_window=self.sliding_window_size, cp_pg=self.cp_pg, position_ids=position_ids, doc_masking=doc_masking,
            flex_attention_mask=getattr(self.config, "flex_attention_mask", None),
        )
        out = self.o_proj(out.reshape(T, self.local_q_size))
        return {"hidden_states": out, "position_ids": position_ids}


class Qwen2DecoderLayer(nn.Module):
    def __init__(self, config, parallel_config: Optional[ParallelismArgs], tp_pg: dist.ProcessGroup, cp_pg: Optional[dist.ProcessGroup], layer_idx: int, parallel_context: Optional[ParallelContext] = None):
        super().__init__()
        self.input_layernorm = TritonRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.attn = Qwen2Attention(config, parallel_config, tp_pg, cp_pg, layer_idx)
        self.post_attention_layernorm = TritonRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        moe = getattr(config, "moe_config", None)
        if moe is not None and layer_idx in moe.layers:
            from nanotron_b200.nn.moe import Qwen2MoELayer

            self.mlp = Qwen2MoELayer(config, parallel_config, tp_pg=tp_pg, ep_pg=parallel_context.ep_pg if parallel_context is not None else None, layer_idx=layer_idx)
            self.is_moe = True
        else:
            self.mlp = Qwen2MLP(config, parallel_config, tp_pg)
            self.is_moe = False
        self.recompute_layer = parallel_config.recompute_layer if parallel_config is not None else False
        self.use_doc_masking = getattr(config, "_use_doc_masking", False)

    def _core_forward(self, hidden_states, position_ids, cu_seqlens=None):
        normed, residual = self.input_layernorm(hidden_states, prenorm=True)
        attn_out = self.attn(hidden_states=normed, position_ids=position_ids, cu_seqlens=cu_seqlens)["hidden_states"]
        normed, residual = self.post_attention_layernorm(attn_out, residual=residual)
        mlp_out = self.mlp(hidden_states=normed)
        hidden_states = mlp_out["hidden_states"] + residual
        return hidden_states, mlp_out.get("aux_loss")

    def forward(self, hidden_states, position_ids, aux_loss=None):
        cu_seqlens = None
        if self.use_doc_masking:
            _, cu_seqlens = get_attention_mask(position_ids, position_ids.shape[1])
        if self.recompute_layer and not isinstance(hidden_states, TensorPointer) and torch.is_grad_enabled():
            hidden_states, layer_aux = checkpoint(self._core_forward, hidden_states, position_ids, cu_seqlens, use_reentrant=False)
        else:
            hidden_states, layer_aux = self._core_forward(hidden_states, position_ids, cu_seqlens)
        out = {"hidden_states": hidden_states, "position_ids": position_ids}
        if aux_loss is not None:
            out["aux_loss"] = aux_loss + layer_aux if layer_aux is not None else aux_loss
        return out


class Embedding(nn.Module):
    def __init__(self, tp_pg: dist.ProcessGroup, config, parallel_config: Optional[ParallelismArgs]):
        super().__init__()
        self.token_embedding = TensorParallelEmbedding(
            num_embeddings=config.vocab_size, embedding_dim=config.hidden_size, padding_idx=config.pad_token_id, pg=tp_pg,
            mode=parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE,
        )
        self.pg = tp_pg
        self.is_moe = getattr(config, "is_moe_model", False)

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor):
        """input_ids: [b, s] -> hidden [b*s (/tp under SP), h]."""
        hidden = self.token_embedding(input_ids.reshape(-1))
        out = {"input_embeds": hidden, "position_ids": position_ids}
        if self.is_moe:
            out["aux_loss"] = torch.zeros((), dtype=torch.float32, device=hidden.device)
        return out


class Qwen2Model(nn.Module):
    """Pipeline graph: embedding -> decoder layers -> final norm -> lm_head (-> fp32 cast is folded into the loss)."""

    def __init__(self, config: Qwen2Config, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs]):
        super().__init__()
        self.p2p = P2P(parallel_context.pp_pg, device=parallel_context.device)
        self.config = config
        self.parallel_config = parallel_config
        self.parallel_context = parallel_context
        self.tp_mode = parallel_config.tp_mode if parallel_config is not None else TensorParallelLinearMode.ALL_REDUCE
        tp_linear_async = parallel_config.tp_linear_async_communication if parallel_config is not None else False
        self.is_moe = getattr(config, "is_moe_model", False)
        extra = {"aux_loss"} if self.is_moe else set()
        self.token_position_embeddings = PipelineBlock(
            p2p=self.p2p, module_builder=Embedding,
            module_kwargs={"tp_pg": parallel_context.tp_pg, "config": config, "parallel_config": parallel_config},
            module_input_keys={"input_ids", "position_ids"}, module_output_keys={"input_embeds", "position_ids"} | extra,
        )
        self.decoder = nn.ModuleList(
            [
                PipelineBlock(
                    p2p=self.p2p, module_builder=self._decoder_layer_class(),
                    module_kwargs={"config": config, "parallel_config": parallel_config, "tp_pg": parallel_context.tp_pg, "cp_pg": parallel_context.cp_pg, "layer_idx": i, "parallel_context": parallel_context},
                    module_input_keys={"hidden_states", "position_ids"} | extra, module_output_keys={"hidden_states", "position_ids"} | extra,
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

    @staticmethod
    def _decoder_layer_class():
        return Qwen2DecoderLayer

    def forward(self, input_ids: Union[torch.Tensor, TensorPointer], position_ids: Union[torch.Tensor, TensorPointer]):
        out = self.token_position_embeddings(input_ids=input_ids, position_ids=position_ids)
        state = {"hidden_states": out["input_embeds"], "position_ids": out["position_ids"]}
        if self.is_moe:
            state["aux_loss"] = out["aux_loss"]
        for layer in self.decoder:
            state = layer(**state)
        hidden = self.final_layer_norm(input=state["hidden_states"])["hidden_states"]
        logits = self.lm_head(x=hidden)["logits"]
        if self.is_moe:
            return logits, state["aux_loss"]
        return logits

    def get_block_compute_costs(self):
        """FLOPs-proportional cost per block class, used to balance pipeline stages."""
        c = self.config
        d_qkv = c.hidden_size // c.num_attention_heads
        inter = c.intermediate_size
        moe = getattr(c, "moe_config", None)
        if moe is not None:
            inter = moe.moe_intermediate_size * moe.top_k + (moe.shared_expert_intermediate_size if moe.enable_shared_expert else 0)
        return {
            self._decoder_layer_class(): 2 * c.num_attention_heads * d_qkv * c.hidden_size
            + 2 * c.num_key_value_heads * d_qkv * c.hidden_size
            + 3 * inter * c.hidden_size,
            TensorParallelColumnLinear: c.vocab_size * c.hidden_size,
        }

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        world = self.parallel_context.world_pg.size()
        c = self.config
        moe = getattr(c, "moe_config", None)
        moe_layers = 0
        if moe is not None:
            moe_layers = c.num_hidden_layers if -1 in moe.layers else len([i for i in moe.layers if 0 <= i < c.num_hidden_layers])
        model_flops, hardware_flops = get_flops(
            num_layers=c.num_hidden_layers, hidden_size=c.hidden_size, num_heads=c.num_attention_heads,
            num_key_value_heads=c.num_key_value_heads, vocab_size=c.vocab_size, ffn_hidden_size=c.intermediate_size,
            seq_len=sequence_length, batch_size=global_batch_size, moe_config=moe, num_moe_layers=moe_layers,
            recompute_layer=bool(getattr(self.parallel_config, "recompute_layer", False)),
        )
        return model_flops / (iteration_time_in_sec * world * 1e12), hardware_flops / (iteration_time_in_sec * world * 1e12)


def masked_mean(loss, label_mask, dtype):
    return (loss * label_mask).sum(dtype=dtype) / label_mask.sum().clamp(min=1)


class Loss(nn.Module):
    def __init__(self, tp_pg: dist.ProcessGroup):
        super().__init__()
        self.tp_pg = tp_pg

    def forward(self, sharded_logits: torch.Tensor, label_ids: torch.Tensor, label_mask: torch.Tensor) -> Dict[str, torch.Tensor]:
        """sharded_logits: [b*s, V/tp]; label_ids/label_mask: [b, s]."""
        loss = sharded_cross_entropy(sharded_logits, label_ids.reshape(-1).contiguous(), group=self.tp_pg, dtype=torch.float)
        return {"loss": masked_mean(loss, label_mask.reshape(-1), dtype=torch.float)}


class LossWithZLoss(Loss):
    def __init__(self, tp_pg: dist.ProcessGroup, z_loss_coefficient: float):
        super().__init__(tp_pg)
        self.z_loss_coef = z_loss_coefficient

    def forward(self, sharded_logits, label_ids, label_mask):
        loss, z = sharded_cross_entropy_with_z_loss(sharded_logits, label_ids.reshape(-1).contiguous(), group=self.tp_pg, dtype=torch.float, z_loss_coef=self.z_loss_coef)
        m = label_mask.reshape(-1)
        z_loss = masked_mean(z.detach(), m, dtype=torch.float)
        return {"loss": masked_mean(loss + z, m, dtype=torch.float), "z_loss": z_loss}


class MoELoss(nn.Module):
    """CE (+ optional z-loss) plus ``router_aux_loss_coef * sum over layers of E * sum_e f_e * P_e``."""

    def __init__(self, tp_pg, aux_coef: float, z_loss_coefficient: Optional[float]):
        super().__init__()
        self.inner = LossWithZLoss(tp_pg, z_loss_coefficient) if z_loss_coefficient else Loss(tp_pg)
        self.aux_coef = aux_coef

    def forward(self, sharded_logits, label_ids, label_mask, aux_loss):
        out = self.inner(sharded_logits, label_ids, label_mask)
        out["aux_loss"] = aux_loss.detach()
        out["loss"] = out["loss"] + self.aux_coef * aux_loss
        return out


class Qwen2ForTraining(NanotronModel):
    model_class = Qwen2Model

    def __init__(self, config: Qwen2Config, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs], random_states: Optional[RandomStates] = None):
        super().__init__()
        self.model = self.model_class(config=config, parallel_context=parallel_context, parallel_config=parallel_config)
        self.is_moe = getattr(config, "is_moe_model", False)
        z = config.z_loss_coefficient if getattr(config, "z_loss_enabled", False) else None
        if self.is_moe:
            self.loss = PipelineBlock(
                p2p=self.model.p2p, module_builder=MoELoss,
                module_kwargs={"tp_pg": parallel_context.tp_pg, "aux_coef": config.moe_config.router_aux_loss_coef, "z_loss_coefficient": z},
                module_input_keys={"sharded_logits", "label_ids", "label_mask", "aux_loss"},
                module_output_keys={"loss", "aux_loss"} | ({"z_loss"} if z else set()),
            )
        elif z:
            self.loss = PipelineBlock(
                p2p=self.model.p2p, module_builder=LossWithZLoss, module_kwargs={"tp_pg": parallel_context.tp_pg, "z_loss_coefficient": z},
                module_input_keys={"sharded_logits", "label_ids", "label_mask"}, module_output_keys={"loss", "z_loss"},
            )
        else:
            self.loss = PipelineBlock(
                p2p=self.model.p2p, module_builder=Loss, module_kwargs={"tp_pg": parallel_context.tp_pg},
                module_input_keys={"sharded_logits", "label_ids", "label_mask"}, module_output_keys={"loss"},
            )
        self.parallel_context = parallel_context
        self.config = config
        self.parallel_config = parallel_config

    def forward(self, input_ids, position_ids, label_ids, label_mask) -> Dict[str, Union[torch.Tensor, TensorPointer]]:
        out = self.model(input_ids=input_ids, position_ids=position_ids)
        if self.is_moe:
            logits, aux = out
            return self.loss(sharded_logits=logits, label_ids=label_ids, label_mask=label_mask, aux_loss=aux)
        return self.loss(sharded_logits=out, label_ids=label_ids, label_mask=label_mask)

    @torch.no_grad()
    def init_model_randomly(self, config: Config):
        init_method = config.model.init_method
        if isinstance(init_method, RandomInit):
            parametrizator_cls = StandardParametrizator
        elif isinstance(init_method, SpectralMupInit):
            parametrizator_cls = SpectralMupParametrizator
        else:
            raise ValueError(f"Unknown init method {init_method}")
        parametrizator = parametrizator_cls(config=config)
        initialized = set()
        module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in self.named_modules()}
        module_id_to_prefix[id(self)] = ""
        for param_name, param in sorted(self.named_parameters(), key=lambda x: x[0]):
            assert isinstance(param, NanotronParameter), f"{param_name} is not a NanotronParameter"
            module_name, _, local_name = param_name.rpartition(".")
            full_name = param.get_tied_info().get_full_name_from_module_id_to_prefix(module_id_to_prefix) if param.is_tied else param_name
            if full_name in initialized:
                continue
            parametrizator.parametrize(param_name, self.get_submodule(module_name))
            initialized.add(full_name)

    def get_embeddings_lm_head_tied_names(self):
        if self.config.tie_word_embeddings:
            return ["model.token_position_embeddings.pp_block.token_embedding.weight", "model.lm_head.pp_block.weight"]
        return []

    def get_block_compute_costs(self):
        return self.model.get_block_compute_costs()

    def get_flops_per_sec(self, iteration_time_in_sec, sequence_length, global_batch_size):
        return self.model.get_flops_per_sec(iteration_time_in_sec, sequence_length, global_batch_size)


def get_flops(num_layers, hidden_size, num_heads, num_key_value_heads, vocab_size, seq_len, ffn_hidden_size, batch_size=1, moe_config=None, num_moe_layers=0, recompute_layer=False):
    """FLOPs of one forward+backward over ``batch_size`` sequences, counted the way the reference does
    (reference src/nanotron/models/qwen.py:1024-1091): full S^2 attention without causal discount, gated MLP
    (3 matrices), lm head; backward = 2 x forward.

    Beyond the reference: a mixture-of-experts layer counts the experts a token actually visits (``top_k`` gated MLPs of
    ``moe_intermediate_size``, the router, and the shared expert with its gate when enabled) instead of a dense MLP, and the
    hardware figure adds the second forward of every decoder layer under full-layer recomputation.
    Returns (model_flops, hardware_flops)."""
    head_dim = hidden_size // num_heads
    T = batch_size * seq_len
    qkv = 2 * T * hidden_size * (num_heads + 2 * num_key_value_heads) * head_dim
    qk = 2 * num_heads * T * seq_len * head_dim
    pv = 2 * num_heads * T * seq_len * head_dim
    out = 2 * T * num_heads * head_dim * hidden_size
    attention = qkv + qk + pv + out
    dense_mlp = 6 * T * hidden_size * ffn_hidden_size
    moe_mlp = 0
    if moe_config is not None and num_moe_layers > 0:
        moe_mlp = 6 * T * hidden_size * moe_config.moe_intermediate_size * moe_config.top_k + 2 * T * hidden_size * moe_config.num_experts
        if moe_config.enable_shared_expert:
            moe_mlp += 6 * T * hidden_size * moe_config.shared_expert_intermediate_size + 2 * T * hidden_size
    layers_fwd = num_layers * attention + (num_layers - num_moe_layers) * dense_mlp + num_moe_layers * moe_mlp
    lm_head = 2 * T * hidden_size * vocab_size
    model_flops = 3 * (layers_fwd + lm_head)
    hardware_flops = model_flops + (layers_fwd if recompute_layer else 0)
    return model_flops, hardware_flops
