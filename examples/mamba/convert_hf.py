"""Hugging Face Mamba checkpoints <-> checkpoints of this framework
(capability parity: reference examples/mamba/convert_hf_to_nanotron.py and convert_nanotron_to_hf.py).

    python examples/mamba/convert_hf.py to-nanotron --checkpoint_path state-spaces/mamba-130m-hf --save_path checkpoints/mamba-130m
    python examples/mamba/convert_hf.py to-hf --checkpoint_path checkpoints/mamba-130m --save_path hf/mamba-130m

The two models store the same tensors under different names; nothing is transposed or re-packed (the in-projection is
[x ; z], the x-projection yields [dt ; B ; C] in both).  The converted checkpoint is a single shard that resumes under any
tensor / pipeline layout.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Dict

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from config import MambaModelConfig  # noqa: E402

_MIXER = ("A_log", "D", "conv1d.weight", "conv1d.bias", "in_proj.weight", "in_proj.bias", "x_proj.weight", "dt_proj.weight", "dt_proj.bias", "out_proj.weight", "out_proj.bias")


def config_from_hf(hf_config) -> MambaModelConfig:
    return MambaModelConfig(
        d_model=hf_config.hidden_size, num_hidden_layers=hf_config.num_hidden_layers, vocab_size=hf_config.vocab_size, pad_vocab_size_multiple=1,
        ssm_cfg={
            "d_state": hf_config.state_size, "d_conv": hf_config.conv_kernel, "expand": hf_config.expand, "dt_rank": hf_config.time_step_rank,
            "dt_min": hf_config.time_step_min, "dt_max": hf_config.time_step_max, "dt_init": hf_config.time_step_init_scheme, "dt_scale": hf_config.time_step_scale,
            "dt_init_floor": hf_config.time_step_floor, "conv_bias": hf_config.use_conv_bias, "bias": hf_config.use_bias,
        },
        rms_norm=True, residual_in_fp32=hf_config.residual_in_fp32, rms_norm_eps=hf_config.layer_norm_epsilon, pad_token_id=hf_config.pad_token_id,
        bos_token_id=hf_config.bos_token_id, eos_token_id=hf_config.eos_token_id, tie_word_embeddings=hf_config.tie_word_embeddings,
    )


def config_to_hf(cfg: MambaModelConfig):
    from transformers import MambaConfig

    c = cfg.ssm()
    return MambaConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.d_model, state_size=c["d_state"], num_hidden_layers=cfg.num_hidden_layers, layer_norm_epsilon=cfg.rms_norm_eps,
        pad_token_id=cfg.pad_token_id, bos_token_id=cfg.bos_token_id, eos_token_id=cfg.eos_token_id, expand=c["expand"], conv_kernel=c["d_conv"], use_bias=c["bias"],
        use_conv_bias=c["conv_bias"], residual_in_fp32=cfg.residual_in_fp32, time_step_rank=c["dt_rank"], time_step_scale=c["dt_scale"], time_step_min=c["dt_min"],
        time_step_max=c["dt_max"], time_step_init_scheme=c["dt_init"], time_step_floor=c["dt_init_floor"], tie_word_embeddings=cfg.tie_word_embeddings,
    )


def _pairs(cfg: MambaModelConfig):
    """(name in this framework, name in Hugging Face) for every tensor."""
    yield "model.token_position_embeddings.pp_block.token_embedding.weight", "backbone.embeddings.weight"
    for i in range(cfg.num_hidden_layers):
        yield f"model.decoder.{i}.pp_block.norm.weight", f"backbone.layers.{i}.norm.weight"
        for t in _MIXER:
            yield f"model.decoder.{i}.pp_block.mixer.{t}", f"backbone.layers.{i}.mixer.{t}"
    yield "model.final_layer_norm.pp_block.weight", "backbone.norm_f.weight"
    yield "model.lm_head.pp_block.weight", "lm_head.weight"


def hf_state_to_nanotron(hf_state: Dict[str, torch.Tensor], cfg: MambaModelConfig) -> Dict[str, torch.Tensor]:
    out = {}
    for ours, theirs in _pairs(cfg):
        if theirs in hf_state:
            out[ours] = hf_state[theirs]
        elif theirs == "lm_head.weight":  # tied models store the matrix once
            out[ours] = hf_state["backbone.embeddings.weight"]
    return out


def nanotron_state_to_hf(state: Dict[str, torch.Tensor], cfg: MambaModelConfig) -> Dict[str, torch.Tensor]:
    return {theirs: state[ours] for ours, theirs in _pairs(cfg) if ours in state}


def build_single_process_model(cfg: MambaModelConfig, dtype=torch.float32, device="cpu"):
    """A ``MambaForTraining`` on one process (tp = pp = dp = 1) with empty weights, plus its parallel context."""
    from mamba import MambaForTraining

    from nanotron_b200.config import ParallelismArgs
    from nanotron_b200.models.base import build_model
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.trainer import mark_tied_parameters

    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29613")):
        os.environ.setdefault(k, v)
    ctx = ParallelContext(1, 1, 1)
    par = ParallelismArgs(dp=1, pp=1, tp=1, tp_mode="ALL_REDUCE", tp_linear_async_communication=False)
    model = build_model(model_builder=lambda: MambaForTraining(config=cfg, parallel_context=ctx, parallel_config=par), parallel_context=ctx, dtype=dtype, device=torch.device(device))
    mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=par)
    return model, ctx


def load_state_into(model, state: Dict[str, torch.Tensor]):
    with torch.no_grad():
        named = dict(model.named_parameters())
        missing = [k for k in named if k not in state]
        assert not missing, f"missing weights: {missing[:5]}"
        for k, p in named.items():
            p.copy_(state[k].to(p.dtype))


def to_nanotron(checkpoint_path: str, save_path: str, dtype=torch.float32):
    from transformers import MambaForCausalLM

    from nanotron_b200.serialize.weights import save_weights

    hf = MambaForCausalLM.from_pretrained(checkpoint_path, torch_dtype=dtype)
    cfg = config_from_hf(hf.config)
    model, ctx = build_single_process_model(cfg, dtype=dtype)
    load_state_into(model, hf_state_to_nanotron(hf.state_dict(), cfg))
    out = Path(save_path)
    out.mkdir(parents=True, exist_ok=True)
    save_weights(model=model, parallel_context=ctx, root_folder=out)
    with open(out / "model_config.json", "w") as f:
        json.dump({k: v for k, v in vars(cfg).items() if not k.startswith("_")}, f, indent=2)
    return model, ctx


def to_hf(checkpoint_path: str, save_path: str, dtype=torch.float32):
    from transformers import MambaForCausalLM

    from nanotron_b200.serialize.weights import load_weights

    with open(Path(checkpoint_path) / "model_config.json") as f:
        cfg = MambaModelConfig(**json.load(f))
    model, ctx = build_single_process_model(cfg, dtype=dtype)
    load_weights(model=model, parallel_context=ctx, root_folder=Path(checkpoint_path))
    hf = MambaForCausalLM(config_to_hf(cfg)).to(dtype)
    missing, unexpected = hf.load_state_dict(nanotron_state_to_hf(dict(model.named_parameters()), cfg), strict=False)
    assert not unexpected and all(k == "lm_head.weight" for k in missing), (missing, unexpected)
    hf.save_pretrained(save_path)
    return hf


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("direction", choices=["to-nanotron", "to-hf"])
    ap.add_argument("--checkpoint_path", required=True)
    ap.add_argument("--save_path", required=True)
    a = ap.parse_args()
    (to_nanotron if a.direction == "to-nanotron" else to_hf)(a.checkpoint_path, a.save_path)
    print(f"saved to {a.save_path}")
