"""Hugging Face Llama checkpoint -> checkpoint of this framework (single shard; resume with any topology).

    python examples/llama/convert_hf_to_nanotron.py --checkpoint_path meta-llama/Llama-3.2-1B --save_path checkpoints/llama-1b
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from convert_weights import build_single_process_model, hf_state_to_nanotron, load_state_into, nanotron_config_from_hf  # noqa: E402


def convert(checkpoint_path: str, save_path: str, dtype=torch.bfloat16):
    from transformers import AutoModelForCausalLM

    from nanotron_b200.serialize.weights import save_weights

    hf = AutoModelForCausalLM.from_pretrained(checkpoint_path, torch_dtype=dtype)
    nt_config = nanotron_config_from_hf(hf.config)
    model, ctx = build_single_process_model(nt_config, dtype=dtype)
    load_state_into(model, hf_state_to_nanotron(hf.state_dict(), nt_config))
    out = Path(save_path)
    out.mkdir(parents=True, exist_ok=True)
    save_weights(model=model, parallel_context=ctx, root_folder=out)
    with open(out / "model_config.json", "w") as f:
        json.dump({k: v for k, v in vars(nt_config).items() if not k.startswith("_") and isinstance(v, (int, float, str, bool, type(None)))}, f, indent=2)
    return model, ctx


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint_path", required=True)
    ap.add_argument("--save_path", required=True)
    a = ap.parse_args()
    convert(a.checkpoint_path, a.save_path)
    print(f"saved to {a.save_path}")
