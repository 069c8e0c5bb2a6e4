"""Weight and config mapping between Hugging Face ``LlamaForCausalLM`` and this framework's ``LlamaForTraining``
(capability parity: reference examples/llama/convert_weights.py).

Names: HF keeps q / k / v and gate / up as separate matrices, here they are fused (``attn.qkv_proj`` = [q; k; v] rows,
``mlp.gate_up_proj`` = [gate; up] rows).  Both sides use the half-rotation RoPE layout when ``rope_interleaved`` is False, so no
permutation of the q / k rows is needed in that case; with ``rope_interleaved`` True the q / k rows are permuted between the
"pairs adjacent" and "halves" conventions.
"""
from __future__ import annotations

from typing import Dict

import torch

HF_TO_NT_CONFIG = {
    "bos_token_id": "bos_token_id", "eos_token_id": "eos_token_id", "hidden_act": "hidden_act", "hidden_size": "hidden_size",
    "initializer_range": "initializer_range", "intermediate_size": "intermediate_size", "max_position_embeddings": "max_position_embeddings",
    "num_attention_heads": "num_attention_heads", "num_hidden_layers": "num_hidden_layers", "num_key_value_heads": "num_key_value_heads",
    "pad_token_id": "pad_token_id", "rms_norm_eps": "rms_norm_eps", "rope_theta": "rope_theta", "tie_word_embeddings": "tie_word_embeddings",
    "vocab_size": "vocab_size",
}


def nanotron_config_from_hf(hf_config, **overrides):
    from nanotron_b200.config import LlamaConfig

    kw = {nt: getattr(hf_config, hf) for hf, nt in HF_TO_NT_CONFIG.items() if getattr(hf_config, hf, None) is not None or hf in ("pad_token_id",)}
    if kw.get("rope_theta") is None:
        params = getattr(hf_config, "rope_parameters", None) or {}
        kw["rope_theta"] = params.get("rope_theta", 10000.0)
    kw.setdefault("rope_interleaved", False)
    scaling = _rope_scaling_of(hf_config)
    if scaling is not None:
        kw["rope_scaling"] = scaling
    kw.update(overrides)
    return LlamaConfig(**{k: v for k, v in kw.items() if v is not None or k == "pad_token_id"})


def _rope_scaling_of(hf_config):
    """The frequency-scaling rule of a Hugging Face configuration (``rope_scaling`` of older releases, ``rope_parameters`` of
    newer ones) without the base frequency; None for plain rotary embeddings."""
    params = getattr(hf_config, "rope_scaling", None) or getattr(hf_config, "rope_parameters", None)
    if not params:
        return None
    rule = {k: v for k, v in dict(params).items() if k != "rope_theta"}
    kind = rule.get("rope_type", rule.get("type", "default"))
    return None if kind in (None, "default") else {**rule, "rope_type": kind}


def hf_config_from_nanotron(nt_config):
    from transformers import LlamaConfig as HFLlamaConfig

    kw = {hf: getattr(nt_config, nt) for hf, nt in HF_TO_NT_CONFIG.items() if hasattr(nt_config, nt)}
    if getattr(nt_config, "rope_scaling", None):
        kw["rope_scaling"] = dict(nt_config.rope_scaling)
    return HFLlamaConfig(**kw, attention_bias=False, mlp_bias=False)


def _permute_rope_rows(w: torch.Tensor, n_heads: int, to_interleaved: bool) -> torch.Tensor:
    """Reorder the rows of a q / k projection between the halves layout [x0..x_{d/2-1} | x_{d/2}..] and the interleaved one."""
    d = w.shape[0] // n_heads
    w = w.view(n_heads, d, -1)
    if to_interleaved:
        w = w.view(n_heads, 2, d // 2, -1).transpose(1, 2)
    else:
        w = w.view(n_heads, d // 2, 2, -1).transpose(1, 2)
    return w.reshape(n_heads * d, -1)


def hf_state_to_nanotron(hf: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    out = {
        "model.token_position_embeddings.pp_block.token_embedding.weight": hf["model.embed_tokens.weight"],
        "model.final_layer_norm.pp_block.weight": hf["model.norm.weight"],
        "model.lm_head.pp_block.weight": hf.get("lm_head.weight", hf["model.embed_tokens.weight"]),
    }
    for i in range(config.num_hidden_layers):
        h, n = f"model.layers.{i}", f"model.decoder.{i}.pp_block"
        q, k, v = (hf[f"{h}.self_attn.{x}_proj.weight"] for x in "qkv")
        if config.rope_interleaved:
            q = _permute_rope_rows(q, config.num_attention_heads, True)
            k = _permute_rope_rows(k, config.num_key_value_heads, True)
        out[f"{n}.attn.qkv_proj.weight"] = torch.cat([q, k, v], dim=0)
        out[f"{n}.attn.o_proj.weight"] = hf[f"{h}.self_attn.o_proj.weight"]
        out[f"{n}.mlp.gate_up_proj.weight"] = torch.cat([hf[f"{h}.mlp.gate_proj.weight"], hf[f"{h}.mlp.up_proj.weight"]], dim=0)
        out[f"{n}.mlp.down_proj.weight"] = hf[f"{h}.mlp.down_proj.weight"]
        out[f"{n}.input_layernorm.weight"] = hf[f"{h}.input_layernorm.weight"]
        out[f"{n}.post_attention_layernorm.weight"] = hf[f"{h}.post_attention_layernorm.weight"]
    return out


def nanotron_state_to_hf(nt: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    hd = config.hidden_size // config.num_attention_heads
    nq, nkv = config.num_attention_heads * hd, config.num_key_value_heads * hd
    out = {
        "model.embed_tokens.weight": nt["model.token_position_embeddings.pp_block.token_embedding.weight"],
        "model.norm.weight": nt["model.final_layer_norm.pp_block.weight"],
    }
    if not config.tie_word_embeddings:
        out["lm_head.weight"] = nt["model.lm_head.pp_block.weight"]
    for i in range(config.num_hidden_layers):
        h, n = f"model.layers.{i}", f"model.decoder.{i}.pp_block"
        q, k, v = torch.split(nt[f"{n}.attn.qkv_proj.weight"], [nq, nkv, nkv], dim=0)
        if config.rope_interleaved:
            q = _permute_rope_rows(q.contiguous(), config.num_attention_heads, False)
            k = _permute_rope_rows(k.contiguous(), config.num_key_value_heads, False)
        out[f"{h}.self_attn.q_proj.weight"], out[f"{h}.self_attn.k_proj.weight"], out[f"{h}.self_attn.v_proj.weight"] = q, k, v
        out[f"{h}.self_attn.o_proj.weight"] = nt[f"{n}.attn.o_proj.weight"]
        gate, up = torch.chunk(nt[f"{n}.mlp.gate_up_proj.weight"], 2, dim=0)
        out[f"{h}.mlp.gate_proj.weight"], out[f"{h}.mlp.up_proj.weight"] = gate, up
        out[f"{h}.mlp.down_proj.weight"] = nt[f"{n}.mlp.down_proj.weight"]
        out[f"{h}.input_layernorm.weight"] = nt[f"{n}.input_layernorm.weight"]
        out[f"{h}.post_attention_layernorm.weight"] = nt[f"{n}.post_attention_layernorm.weight"]
    return out


def build_single_process_model(nt_config, dtype=torch.float32, device="cpu"):
    """A ``LlamaForTraining`` on one process (tp = pp = dp = 1) with empty weights, plus its parallel context."""
    import os

    from nanotron_b200.config import ParallelismArgs
    from nanotron_b200.models.base import build_model
    from nanotron_b200.models.llama import LlamaForTraining
    from nanotron_b200.parallel import ParallelContext

    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29611")):
        os.environ.setdefault(k, v)
    ctx = ParallelContext(1, 1, 1)
    par = ParallelismArgs(dp=1, pp=1, tp=1)
    model = build_model(model_builder=lambda: LlamaForTraining(config=nt_config, parallel_context=ctx, parallel_config=par, random_states=None),
                        parallel_context=ctx, dtype=dtype, device=torch.device(device))
    from nanotron_b200.trainer import mark_tied_parameters

    mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=par)  # tied embeddings + replicated (norm) weights get their metadata
    return model, ctx


def load_state_into(model, state: Dict[str, torch.Tensor]):
    with torch.no_grad():
        named = dict(model.named_parameters())
        missing = [k for k in named if k not in state]
        assert not missing, f"missing weights: {missing[:5]}"
        for k, p in named.items():
            p.copy_(state[k].to(p.dtype))
