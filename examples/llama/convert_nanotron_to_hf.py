"""Checkpoint of this framework (Llama) -> Hugging Face ``LlamaForCausalLM`` folder.

    python examples/llama/convert_nanotron_to_hf.py --checkpoint_path checkpoints/10 --save_path hf_out [--tokenizer_name NAME]
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from convert_weights import build_single_process_model, hf_config_from_nanotron, nanotron_state_to_hf  # noqa: E402


def convert(checkpoint_path: str, save_path: str, tokenizer_name=None, dtype=torch.bfloat16):
    from transformers import AutoTokenizer, LlamaForCausalLM

    from nanotron_b200.config import LlamaConfig
    from nanotron_b200.serialize.weights import load_weights

    ckpt = Path(checkpoint_path)
    with open(ckpt / "model_config.json") as f:
        raw = json.load(f)
    fields = {f for f in LlamaConfig.__dataclass_fields__}
    nt_config = LlamaConfig(**{k: v for k, v in raw.items() if k in fields})
    model, ctx = build_single_process_model(nt_config, dtype=dtype)
    load_weights(model=model, parallel_context=ctx, root_folder=ckpt)  # merges tensor-parallel shards written by any topology
    hf = LlamaForCausalLM(hf_config_from_nanotron(nt_config)).to(dtype)
    state = nanotron_state_to_hf({k: v.detach() for k, v in model.named_parameters()}, nt_config)
    missing, unexpected = hf.load_state_dict(state, strict=False)
    assert not unexpected and all("rotary" in m or (nt_config.tie_word_embeddings and m == "lm_head.weight") for m in missing), (missing, unexpected)
    hf.save_pretrained(save_path)
    if tokenizer_name:
        AutoTokenizer.from_pretrained(tokenizer_name).save_pretrained(save_path)
    return hf


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint_path", required=True)
    ap.add_argument("--save_path", required=True)
    ap.add_argument("--tokenizer_name", default=None)
    a = ap.parse_args()
    convert(a.checkpoint_path, a.save_path, a.tokenizer_name)
    print(f"saved to {a.save_path}")
