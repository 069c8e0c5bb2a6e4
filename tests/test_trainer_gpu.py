"""Trainer on one GPU: in-tree kernels are the ones that run, the optimizer takes the single-launch flat path, and the
bf16 loss curve tracks the fp32 PyTorch-oracle curve."""
import pytest
import torch

from helpers import dummy_dataloader, make_config, single_process_env, tiny_llama_config

pytestmark = pytest.mark.gpu


def _run(steps, ops_mode, dtype, seq=128):
    from nanotron_b200 import ops
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    ops.set_mode(ops_mode)
    try:
        cfg = make_config(tiny_llama_config(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, vocab_size=1024), seq=seq, mbs=4, steps=steps, dtype=dtype, lr=1e-3)
        t = DistributedTrainer(cfg)
        t.prepare_training()
        dl = dummy_dataloader(t)
        # one fixed batch repeated: the model must be able to overfit it
        batch = next(dl)
        losses = []
        n0 = ops.native_launches()
        for _ in range(steps):
            _, loss, _ = t.training_step(iter([batch]))
            t.iteration_step += 1
            losses.append(float(loss))
        launches = ops.native_launches() - n0
        base = t.optimizer.get_base_optimizer()
        flat = getattr(base, "_flat", None) is not None
        t.parallel_context.destroy()
        return losses, launches, flat
    finally:
        ops.set_mode("auto")


def test_native_path_runs_and_learns():
    losses, launches, flat = _run(8, "auto", "bfloat16")
    assert launches > 8 * 20, "in-tree kernels did not run"
    assert flat, "optimizer did not take the flat single-launch path"
    assert losses[-1] < losses[0] - 0.5, losses


def test_native_matches_oracle_curve():
    native, _, _ = _run(6, "auto", "bfloat16")
    oracle, _, _ = _run(6, "torch", "float32")
    for a, b in zip(native, oracle):
        assert abs(a - b) < 0.08, (native, oracle)


def _model_losses(model_config, ops_mode, dtype, steps=4, seq=512, mbs=2, ragged_docs=False):
    """Loss curve of a tiny model trained on one fixed batch; ``ragged_docs`` packs documents of unequal length into every row."""
    from nanotron_b200 import ops
    from nanotron_b200.trainer import DistributedTrainer

    single_process_env()
    ops.set_mode(ops_mode)
    try:
        t = DistributedTrainer(make_config(model_config, seq=seq, mbs=mbs, steps=steps, dtype=dtype, lr=1e-3))
        t.prepare_training()
        batch = next(dummy_dataloader(t))
        if ragged_docs:
            lens = [200, 57, 255]
            assert sum(lens) == seq
            pos = torch.cat([torch.arange(n) for n in lens]).to(batch["position_ids"].device)
            pos_rev = torch.cat([torch.arange(n) for n in reversed(lens)]).to(pos.device)
            batch["position_ids"] = torch.stack([pos, pos_rev])[:mbs].contiguous()
        n0 = ops.native_launches()
        losses = []
        for _ in range(steps):
            _, loss, _ = t.training_step(iter([batch]))
            t.iteration_step += 1
            losses.append(float(loss))
        launches = ops.native_launches() - n0
        t.parallel_context.destroy()
        return losses, launches
    finally:
        ops.set_mode("auto")


def test_qwen2_packed_documents_run_the_in_tree_attention():
    """Document masking with ragged documents per row: the default path must be the in-tree kernel and track the fp32 oracle."""
    from helpers import tiny_qwen_config
    from nanotron_b200.ops import native_attn

    def mc():
        c = tiny_qwen_config(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1, vocab_size=1024, max_position_embeddings=512)
        c._use_doc_masking = True
        return c

    calls = {"n": 0}
    orig = native_attn.flash_attn_fwd

    def counting(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native_attn.flash_attn_fwd = counting
    from nanotron_b200.ops import native

    orig_native = native.flash_attn_fwd
    native.flash_attn_fwd = counting
    try:
        got, launches = _model_losses(mc(), "auto", "bfloat16", ragged_docs=True)
    finally:
        native_attn.flash_attn_fwd = orig
        native.flash_attn_fwd = orig_native
    assert calls["n"] >= 4 * 2, "the in-tree attention kernel did not run on packed documents"
    exp, _ = _model_losses(mc(), "torch", "float32", ragged_docs=True)
    for a, b in zip(got, exp):
        assert abs(a - b) < 0.08, (got, exp)


def test_starcoder2_sliding_window_matches_oracle_curve():
    from nanotron_b200.config import Starcoder2Config

    def mc():
        return Starcoder2Config(hidden_size=256, num_attention_heads=2, num_hidden_layers=2, intermediate_size=512, vocab_size=1024, max_position_embeddings=512, multi_query=False, grouped_query=True, num_kv_heads=1, sliding_window_size=128, global_attn_layers=[1], attn_pdrop=0.0, resid_pdrop=0.0, embd_pdrop=0.0, use_rotary_embeddings=True)

    got, launches = _model_losses(mc(), "auto", "bfloat16")
    assert launches > 4 * 10
    exp, _ = _model_losses(mc(), "torch", "float32")
    for a, b in zip(got, exp):
        assert abs(a - b) < 0.08, (got, exp)
    # multi-query variant (one kv head shared by all query heads, kv projection replicated)
    def mq():
        c = mc()
        c.multi_query, c.grouped_query = True, False
        return c

    got, _ = _model_losses(mq(), "auto", "bfloat16")
    exp, _ = _model_losses(mq(), "torch", "float32")
    for a, b in zip(got, exp):
        assert abs(a - b) < 0.08, (got, exp)
