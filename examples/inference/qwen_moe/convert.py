"""Hugging Face ``Qwen2MoeForCausalLM``  <->  this framework's ``Qwen2ForTraining`` with a ``moe_config``
(capability parity: reference examples/inference/qwen_moe/convert.py).

    python examples/inference/qwen_moe/convert.py to-nanotron --hf-path Qwen/Qwen1.5-MoE-A2.7B --out checkpoints/qwen_moe
    python examples/inference/qwen_moe/convert.py to-hf --checkpoint checkpoints/qwen_moe/0 --out hf_out

Layout differences handled here:
  * attention: HF keeps q / k / v (with biases) apart, here they are one ``qkv_proj`` ([q; k; v] rows);
  * routed experts: HF stores ``experts.gate_up_proj`` as [E, 2I, h] and ``experts.down_proj`` as [E, h, I]; here the grouped GEMMs
    read ``merged_gate_up_proj`` [E, h, 2I] and ``merged_down_proj`` [E, I, h] (token rows times weight, no transposes at run time);
  * shared expert: separate gate / up matrices there, fused ``gate_up_proj`` here; the sigmoid gate ``shared_expert_gate`` maps 1:1;
  * the router weight is kept in fp32 here.
Routing semantics match ``norm_topk_prob=False`` (the probabilities of the selected experts are used as they are).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Dict

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))


def nanotron_config_from_hf(hf_config, **overrides):
    from nanotron_b200.config import MoEConfig, Qwen2Config

    assert not getattr(hf_config, "norm_topk_prob", False), "norm_topk_prob=True is not supported (selected probabilities are not re-normalised here)"
    assert getattr(hf_config, "decoder_sparse_step", 1) == 1 and not getattr(hf_config, "mlp_only_layers", []), "mixed dense / sparse layer patterns are not handled by this converter"
    rope_theta = getattr(hf_config, "rope_theta", None)
    if rope_theta is None:
        rope_theta = (getattr(hf_config, "rope_parameters", None) or {}).get("rope_theta", 1000000.0)
    kw = dict(
        hidden_size=hf_config.hidden_size, intermediate_size=hf_config.intermediate_size, num_hidden_layers=hf_config.num_hidden_layers,
        num_attention_heads=hf_config.num_attention_heads, num_key_value_heads=hf_config.num_key_value_heads, vocab_size=hf_config.vocab_size,
        max_position_embeddings=hf_config.max_position_embeddings, rms_norm_eps=hf_config.rms_norm_eps, rope_theta=rope_theta,
        tie_word_embeddings=bool(hf_config.tie_word_embeddings), attention_bias=True, rope_interleaved=False,
        moe_config=MoEConfig(num_experts=hf_config.num_experts, top_k=hf_config.num_experts_per_tok, moe_intermediate_size=hf_config.moe_intermediate_size,
                             shared_expert_intermediate_size=hf_config.shared_expert_intermediate_size, enable_shared_expert=True,
                             router_aux_loss_coef=getattr(hf_config, "router_aux_loss_coef", 0.001)),
    )
    kw.update(overrides)
    return Qwen2Config(**kw)


def hf_config_from_nanotron(nt_config):
    from transformers import Qwen2MoeConfig

    moe = nt_config.moe_config
    return Qwen2MoeConfig(
        vocab_size=nt_config.vocab_size, hidden_size=nt_config.hidden_size, intermediate_size=nt_config.intermediate_size, num_hidden_layers=nt_config.num_hidden_layers,
        num_attention_heads=nt_config.num_attention_heads, num_key_value_heads=nt_config.num_key_value_heads, max_position_embeddings=nt_config.max_position_embeddings,
        rms_norm_eps=nt_config.rms_norm_eps, rope_theta=nt_config.rope_theta, tie_word_embeddings=nt_config.tie_word_embeddings, moe_intermediate_size=moe.moe_intermediate_size,
        shared_expert_intermediate_size=moe.shared_expert_intermediate_size, num_experts=moe.num_experts, num_experts_per_tok=moe.top_k, norm_topk_prob=False,
        decoder_sparse_step=1, mlp_only_layers=[], router_aux_loss_coef=moe.router_aux_loss_coef,
    )


def hf_state_to_nanotron(hf: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    out = {
        "model.token_position_embeddings.pp_block.token_embedding.weight": hf["model.embed_tokens.weight"],
        "model.final_layer_norm.pp_block.weight": hf["model.norm.weight"],
        "model.lm_head.pp_block.weight": hf.get("lm_head.weight", hf["model.embed_tokens.weight"]),
    }
    for i in range(config.num_hidden_layers):
        h, n = f"model.layers.{i}", f"model.decoder.{i}.pp_block"
        out[f"{n}.attn.qkv_proj.weight"] = torch.cat([hf[f"{h}.self_attn.{x}_proj.weight"] for x in "qkv"], dim=0)
        out[f"{n}.attn.qkv_proj.bias"] = torch.cat([hf[f"{h}.self_attn.{x}_proj.bias"] for x in "qkv"], dim=0)
        out[f"{n}.attn.o_proj.weight"] = hf[f"{h}.self_attn.o_proj.weight"]
        out[f"{n}.input_layernorm.weight"] = hf[f"{h}.input_layernorm.weight"]
        out[f"{n}.post_attention_layernorm.weight"] = hf[f"{h}.post_attention_layernorm.weight"]
        out[f"{n}.mlp.router.weight"] = hf[f"{h}.mlp.gate.weight"].float()
        if f"{h}.mlp.experts.gate_up_proj" in hf:  # fused expert tensors
            gate_up, down = hf[f"{h}.mlp.experts.gate_up_proj"], hf[f"{h}.mlp.experts.down_proj"]
        else:  # one module per expert (older checkpoints)
            E = config.moe_config.num_experts
            gate_up = torch.stack([torch.cat([hf[f"{h}.mlp.experts.{e}.gate_proj.weight"], hf[f"{h}.mlp.experts.{e}.up_proj.weight"]], dim=0) for e in range(E)])
            down = torch.stack([hf[f"{h}.mlp.experts.{e}.down_proj.weight"] for e in range(E)])
        out[f"{n}.mlp.experts.merged_gate_up_proj"] = gate_up.transpose(1, 2).contiguous()  # [E, 2I, h] -> [E, h, 2I]
        out[f"{n}.mlp.experts.merged_down_proj"] = down.transpose(1, 2).contiguous()  # [E, h, I] -> [E, I, h]
        out[f"{n}.mlp.shared_expert.gate_up_proj.weight"] = torch.cat([hf[f"{h}.mlp.shared_expert.gate_proj.weight"], hf[f"{h}.mlp.shared_expert.up_proj.weight"]], dim=0)
        out[f"{n}.mlp.shared_expert.down_proj.weight"] = hf[f"{h}.mlp.shared_expert.down_proj.weight"]
        out[f"{n}.mlp.shared_expert_gate.weight"] = hf[f"{h}.mlp.shared_expert_gate.weight"]
    return out


def nanotron_state_to_hf(nt: Dict[str, torch.Tensor], config) -> Dict[str, torch.Tensor]:
    hd = config.hidden_size // config.num_attention_heads
    nq, nkv = config.num_attention_heads * hd, config.num_key_value_heads * hd
    out = {"model.embed_tokens.weight": nt["model.token_position_embeddings.pp_block.token_embedding.weight"], "model.norm.weight": nt["model.final_layer_norm.pp_block.weight"]}
    if not config.tie_word_embeddings:
        out["lm_head.weight"] = nt["model.lm_head.pp_block.weight"]
    for i in range(config.num_hidden_layers):
        h, n = f"model.layers.{i}", f"model.decoder.{i}.pp_block"
        for name, part in zip("qkv", torch.split(nt[f"{n}.attn.qkv_proj.weight"], [nq, nkv, nkv], dim=0)):
            out[f"{h}.self_attn.{name}_proj.weight"] = part
        for name, part in zip("qkv", torch.split(nt[f"{n}.attn.qkv_proj.bias"], [nq, nkv, nkv], dim=0)):
            out[f"{h}.self_attn.{name}_proj.bias"] = part
        out[f"{h}.self_attn.o_proj.weight"] = nt[f"{n}.attn.o_proj.weight"]
        out[f"{h}.input_layernorm.weight"] = nt[f"{n}.input_layernorm.weight"]
        out[f"{h}.post_attention_layernorm.weight"] = nt[f"{n}.post_attention_layernorm.weight"]
        out[f"{h}.mlp.gate.weight"] = nt[f"{n}.mlp.router.weight"]
        out[f"{h}.mlp.experts.gate_up_proj"] = nt[f"{n}.mlp.experts.merged_gate_up_proj"].transpose(1, 2).contiguous()
        out[f"{h}.mlp.experts.down_proj"] = nt[f"{n}.mlp.experts.merged_down_proj"].transpose(1, 2).contiguous()
        gate, up = torch.chunk(nt[f"{n}.mlp.shared_expert.gate_up_proj.weight"], 2, dim=0)
        out[f"{h}.mlp.shared_expert.gate_proj.weight"], out[f"{h}.mlp.shared_expert.up_proj.weight"] = gate, up
        out[f"{h}.mlp.shared_expert.down_proj.weight"] = nt[f"{n}.mlp.shared_expert.down_proj.weight"]
        out[f"{h}.mlp.shared_expert_gate.weight"] = nt[f"{n}.mlp.shared_expert_gate.weight"]
    return out


def build_single_process_model(nt_config, dtype=torch.float32, device="cpu"):
    from nanotron_b200.config import ParallelismArgs
    from nanotron_b200.models.base import build_model
    from nanotron_b200.models.qwen import Qwen2ForTraining
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.trainer import mark_tied_parameters

    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29613")):
        os.environ.setdefault(k, v)
    ctx = ParallelContext(1, 1, 1)
    par = ParallelismArgs(dp=1, pp=1, tp=1)
    model = build_model(model_builder=lambda: Qwen2ForTraining(config=nt_config, parallel_context=ctx, parallel_config=par, random_states=None), parallel_context=ctx, dtype=dtype, device=torch.device(device))
    mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=par)
    return model, ctx


def load_state_into(model, state: Dict[str, torch.Tensor]):
    with torch.no_grad():
        named = dict(model.named_parameters())
        missing = [k for k in named if k not in state]
        assert not missing, f"missing weights: {missing[:5]}"
        for k, p in named.items():
            p.copy_(state[k].to(p.dtype))


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("to-nanotron")
    a.add_argument("--hf-path", required=True)
    a.add_argument("--out", required=True)
    b = sub.add_parser("to-hf")
    b.add_argument("--checkpoint", required=True, help="checkpoint step folder written by this framework")
    b.add_argument("--out", required=True)
    args = ap.parse_args()
    if args.cmd == "to-nanotron":
        from transformers import AutoModelForCausalLM

        from nanotron_b200.serialize.weights import save_weights

        hf = AutoModelForCausalLM.from_pretrained(args.hf_path, torch_dtype=torch.bfloat16)
        cfg = nanotron_config_from_hf(hf.config)
        model, ctx = build_single_process_model(cfg, dtype=torch.bfloat16)
        load_state_into(model, hf_state_to_nanotron(hf.state_dict(), cfg))
        out = Path(args.out) / "0"
        out.mkdir(parents=True, exist_ok=True)
        save_weights(model=model, parallel_context=ctx, root_folder=out)
        from dataclasses import asdict

        (out / "model_config.json").write_text(json.dumps(asdict(cfg), default=str))
        print(f"wrote {out}")
        ctx.destroy()
    else:
        from nanotron_b200.config import MoEConfig, Qwen2Config
        from nanotron_b200.serialize.weights import load_weights

        raw = json.loads((Path(args.checkpoint) / "model_config.json").read_text())
        raw["moe_config"] = MoEConfig(**raw["moe_config"])
        cfg = Qwen2Config(**{k: v for k, v in raw.items() if k in Qwen2Config.__dataclass_fields__})
        model, ctx = build_single_process_model(cfg, dtype=torch.bfloat16)
        load_weights(model=model, parallel_context=ctx, root_folder=Path(args.checkpoint))
        from transformers import Qwen2MoeForCausalLM

        hf = Qwen2MoeForCausalLM(hf_config_from_nanotron(cfg)).to(torch.bfloat16)
        hf.load_state_dict(nanotron_state_to_hf({k: v.detach() for k, v in model.named_parameters()}, cfg), strict=False)
        hf.save_pretrained(args.out)
        print(f"wrote {args.out}")
        ctx.destroy()


if __name__ == "__main__":
    main()
