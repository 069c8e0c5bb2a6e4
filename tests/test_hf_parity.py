"""Numerical parity with Hugging Face ``LlamaForCausalLM``: a random tiny HF model converted with examples/llama gives the
same logits here (fp32, CPU), the conversion round-trips, and a saved checkpoint converts back to an HF folder."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "llama"))

transformers = pytest.importorskip("transformers")


def _tiny_hf(tie=False):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=176, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2,
                      max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=tie, attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval().float()


@pytest.mark.parametrize("interleaved", [False, True])
def test_logits_match_hugging_face(interleaved):
    from convert_weights import build_single_process_model, hf_state_to_nanotron, load_state_into, nanotron_config_from_hf, nanotron_state_to_hf
    from helpers import single_process_env

    single_process_env()
    hf = _tiny_hf()
    nt_cfg = nanotron_config_from_hf(hf.config, rope_interleaved=interleaved)
    model, ctx = build_single_process_model(nt_cfg)
    state = hf_state_to_nanotron(hf.state_dict(), nt_cfg)
    load_state_into(model, state)
    model.eval()
    ids = torch.randint(0, 320, (2, 37))
    with torch.no_grad():
        exp = hf(input_ids=ids).logits
        got = model.model(input_ids=ids, input_mask=torch.ones_like(ids, dtype=torch.bool))
    got = got.reshape(2, 37, -1) if got.dim() == 2 else got
    if got.shape[0] == 37:  # [s, b, v] layout
        got = got.transpose(0, 1)
    torch.testing.assert_close(got.float(), exp, atol=2e-4, rtol=1e-3)
    back = nanotron_state_to_hf(state, nt_cfg)
    for k, v in hf.state_dict().items():
        if "rotary" in k:
            continue
        assert torch.equal(back[k], v), k
    ctx.destroy()


def test_checkpoint_converts_back_to_hf_folder(tmp_path):
    import json

    from convert_nanotron_to_hf import convert as to_hf
    from convert_weights import build_single_process_model, hf_state_to_nanotron, load_state_into, nanotron_config_from_hf
    from helpers import single_process_env
    from nanotron_b200.serialize.weights import save_weights

    single_process_env()
    hf = _tiny_hf()
    nt_cfg = nanotron_config_from_hf(hf.config)
    model, ctx = build_single_process_model(nt_cfg)
    load_state_into(model, hf_state_to_nanotron(hf.state_dict(), nt_cfg))
    ckpt = tmp_path / "nt"
    ckpt.mkdir()
    save_weights(model=model, parallel_context=ctx, root_folder=ckpt)
    with open(ckpt / "model_config.json", "w") as f:
        json.dump({k: v for k, v in vars(nt_cfg).items() if isinstance(v, (int, float, str, bool, type(None)))}, f)
    ctx.destroy()
    single_process_env()
    os.environ["MASTER_PORT"] = str(int(os.environ["MASTER_PORT"]) + 1)
    out = to_hf(str(ckpt), str(tmp_path / "hf"), dtype=torch.float32)
    ids = torch.randint(0, 320, (1, 16))
    with torch.no_grad():
        torch.testing.assert_close(out(input_ids=ids).logits, hf(input_ids=ids).logits, atol=1e-5, rtol=1e-5)
    assert (tmp_path / "hf" / "config.json").exists()
    torch.distributed.destroy_process_group()
