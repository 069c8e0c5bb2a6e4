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


def test_qwen2_moe_logits_match_hugging_face():
    """A random tiny ``Qwen2MoeForCausalLM`` (routed experts + gated shared expert, q / k / v biases) converted with
    examples/inference/qwen_moe gives the same logits here, and the weight mapping round-trips."""
    import importlib.util

    from helpers import single_process_env

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("qwen_moe_convert", os.path.join(root, "examples", "inference", "qwen_moe", "convert.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)
    from transformers import Qwen2MoeConfig, Qwen2MoeForCausalLM

    cfg = Qwen2MoeConfig(vocab_size=160, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=16,
                         shared_expert_intermediate_size=48, num_experts=4, num_experts_per_tok=2, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[],
                         max_position_embeddings=64, tie_word_embeddings=False, rope_theta=10000.0)
    torch.manual_seed(0)
    hf = Qwen2MoeForCausalLM(cfg).eval().float()
    single_process_env()
    nt_cfg = conv.nanotron_config_from_hf(hf.config)
    assert nt_cfg.moe_config.num_experts == 4 and nt_cfg.moe_config.enable_shared_expert and nt_cfg.attention_bias
    model, ctx = conv.build_single_process_model(nt_cfg)
    state = conv.hf_state_to_nanotron(hf.state_dict(), nt_cfg)
    conv.load_state_into(model, state)
    model.eval()
    ids = torch.randint(0, 160, (2, 19))
    pos = torch.arange(19).unsqueeze(0).expand(2, -1).contiguous()
    with torch.no_grad():
        exp = hf(input_ids=ids).logits
        got = model.model(input_ids=ids, position_ids=pos)
    got = got[0] if isinstance(got, tuple) else got
    torch.testing.assert_close(got.float().reshape(2, 19, -1), exp, atol=3e-4, rtol=1e-3)
    back = conv.nanotron_state_to_hf(state, nt_cfg)
    for k, v in hf.state_dict().items():
        if "rotary" in k:
            continue
        assert torch.equal(back[k].to(v.dtype), v), k
    ctx.destroy()


def test_mamba_example_matches_the_hugging_face_model(tmp_path):
    """examples/mamba against transformers' own Mamba (its sequential PyTorch path): same logits from the same weights, and a
    checkpoint that goes Hugging Face -> this framework -> Hugging Face unchanged."""
    import importlib.util
    import os
    import sys

    transformers = pytest.importorskip("transformers")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "examples", "mamba"))
    spec = importlib.util.spec_from_file_location("mamba_convert_hf", os.path.join(root, "examples", "mamba", "convert_hf.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)

    torch.manual_seed(0)
    hf_cfg = transformers.MambaConfig(vocab_size=96, hidden_size=32, state_size=8, num_hidden_layers=2, conv_kernel=4, expand=2, time_step_rank=4, use_mambapy=False,
                                      pad_token_id=0, bos_token_id=1, eos_token_id=2)
    hf = transformers.MambaForCausalLM(hf_cfg).eval()
    hf_dir = tmp_path / "hf"
    hf.save_pretrained(hf_dir)
    model, ctx = conv.to_nanotron(str(hf_dir), str(tmp_path / "nt"))
    ids = torch.randint(3, 96, (2, 24))
    with torch.no_grad():
        want = hf(ids).logits
        got = model.eval().model(input_ids=ids, input_mask=torch.ones(2, 24, dtype=torch.bool)).view(2, 24, -1)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=1e-4)
    ctx.destroy()
    back = conv.to_hf(str(tmp_path / "nt"), str(tmp_path / "hf_back"))
    for name, p in hf.state_dict().items():
        assert torch.equal(back.state_dict()[name], p), name


@pytest.mark.parametrize("kind", ["llama3", "linear"])
def test_rope_frequency_scaling_matches_hugging_face(kind):
    """Llama-3.1 checkpoints carry ``rope_scaling``: the frequencies, and the logits of a converted model at positions beyond the
    original context, must equal the Hugging Face ones."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    from convert_weights import build_single_process_model, hf_config_from_nanotron, hf_state_to_nanotron, load_state_into, nanotron_config_from_hf
    from helpers import single_process_env
    from nanotron_b200.ops.reference import rope_inverse_frequencies

    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32} if kind == "llama3" else {"rope_type": "linear", "factor": 4.0}
    cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256,
                      rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=dict(scaling), attention_bias=False, mlp_bias=False)
    expected, _ = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
    torch.testing.assert_close(rope_inverse_frequencies(32, 10000.0, scaling), expected.float(), rtol=1e-6, atol=0)
    with pytest.raises(NotImplementedError):
        rope_inverse_frequencies(32, 10000.0, {"rope_type": "yarn", "factor": 2.0})
    torch.manual_seed(0)
    hf = LlamaForCausalLM(cfg).eval().float()
    single_process_env()
    nt_cfg = nanotron_config_from_hf(hf.config)
    assert nt_cfg.rope_scaling == scaling
    back = hf_config_from_nanotron(nt_cfg)  # and the rule survives the way back
    assert {k: v for k, v in back.rope_parameters.items() if k != "rope_theta"} == scaling
    model, ctx = build_single_process_model(nt_cfg)
    load_state_into(model, hf_state_to_nanotron(hf.state_dict(), nt_cfg))
    model.eval()
    ids = torch.randint(0, 320, (1, 150))  # well past the original 32 positions
    with torch.no_grad():
        exp = hf(input_ids=ids).logits
        got = model.model(input_ids=ids, input_mask=torch.ones_like(ids, dtype=torch.bool)).reshape(1, 150, -1)
    torch.testing.assert_close(got.float(), exp, atol=3e-4, rtol=1e-3)
    ctx.destroy()
