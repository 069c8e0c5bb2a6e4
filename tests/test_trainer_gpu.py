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
