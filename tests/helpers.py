"""Test helpers: spawn ``world_size`` gloo ranks on CPU and run a function in each
(strategy parity: reference tests/helpers/utils.py init_distributed, which needs one GPU per rank)."""
from __future__ import annotations

import os
import socket
import sys
import tempfile
import traceback
from typing import Callable

import torch
import torch.multiprocessing as mp


_USED_PORTS = set()


def _free_port() -> int:
    """A port for a rendezvous that starts a moment later.  Taken from below the range the kernel hands out to outgoing connections
    (32768 and up on Linux), so that neither the ranks' own connections nor another process can take it in between; each port is
    tried at most once per process."""
    import random

    for _ in range(200):
        port = random.randint(12000, 32000)
        if port in _USED_PORTS:
            continue
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", port))
            except OSError:
                continue
        _USED_PORTS.add(port)
        return port
    raise RuntimeError("no free port found")


def _worker(rank: int, world_size: int, port: int, fn: Callable, kwargs: dict, err_dir: str):
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world_size), "LOCAL_WORLD_SIZE": str(world_size), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    try:
        fn(**kwargs)
    except BaseException:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn: Callable, world_size: int, **kwargs):
    """Run ``fn(**kwargs)`` on ``world_size`` CPU processes with the env vars torchrun would set."""
    port = _free_port()
    with tempfile.TemporaryDirectory() as err_dir:
        try:
            mp.spawn(_worker, args=(world_size, port, fn, kwargs, err_dir), nprocs=world_size, join=True)
        except Exception as e:
            msgs = []
            for name in sorted(os.listdir(err_dir)):
                with open(os.path.join(err_dir, name)) as f:
                    msgs.append(f"--- {name} ---\n{f.read()}")
            raise AssertionError("distributed test failed:\n" + "\n".join(msgs)) from e


def single_process_env():
    """Env for a world_size=1 run inside the test process."""
    os.environ.update({"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "LOCAL_WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(_free_port())})


def tiny_llama_config(**over):
    from nanotron_b200.config import LlamaConfig

    base = dict(hidden_size=16, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, vocab_size=256, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, hidden_act="silu")
    base.update(over)
    return LlamaConfig(**base)


def tiny_qwen_config(**over):
    from nanotron_b200.config import Qwen2Config

    base = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=256, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    base.update(over)
    return Qwen2Config(**base)


def make_config(model_config, tp=1, pp=1, dp=1, cp=1, ep=1, seq=32, mbs=2, accum=1, steps=10, zero=0, fp32_accum=True, dtype="float32", tp_mode="all_reduce", pp_engine="afab", async_tp=False, ckpt_path=None, ckpt_interval=1000, clip=1.0, lr=3e-4, recompute=False, sanity=False):
    import nanotron_b200.config as c

    return c.Config(
        general=c.GeneralArgs(project="test", run="t", seed=42, ignore_sanity_checks=not sanity),
        parallelism=c.ParallelismArgs(dp=dp, pp=pp, tp=tp, pp_engine=pp_engine, tp_mode=tp_mode, tp_linear_async_communication=async_tp, context_parallel_size=cp, expert_parallel_size=ep, recompute_layer=recompute),
        model=c.ModelArgs(model_config=model_config, init_method=c.RandomInit(std=0.025), dtype=dtype),
        tokenizer=c.TokenizerArgs(),
        checkpoints=c.CheckpointsArgs(checkpoints_path=ckpt_path or "/tmp/ntb_ckpt_unused", checkpoint_interval=ckpt_interval, save_final_state=False),
        logging=c.LoggingArgs(log_level="warning", log_level_replica="warning"),
        tokens=c.TokensArgs(sequence_length=seq, train_steps=steps, micro_batch_size=mbs, batch_accumulation_per_replica=accum),
        optimizer=c.OptimizerArgs(
            optimizer_factory=c.AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=False),
            zero_stage=zero, weight_decay=0.01, clip_grad=clip, accumulate_grad_in_fp32=fp32_accum,
            learning_rate_scheduler=c.LRSchedulerArgs(learning_rate=lr, lr_warmup_steps=0, lr_decay_style="cosine", min_decay_lr=lr * 0.1),
        ),
        data_stages=[c.DatasetStageArgs(name="stable", start_training_step=1, data=c.DataArgs(dataset=None, seed=42, num_loading_workers=0))],
    )


def dummy_dataloader(trainer):
    from nanotron_b200.data.dataloader import dummy_infinite_data_generator
    from nanotron_b200.config import LlamaConfig, Starcoder2Config

    cfg = trainer.config
    uses_mask = isinstance(trainer.model_config, (LlamaConfig, Starcoder2Config))
    return dummy_infinite_data_generator(
        micro_batch_size=cfg.tokens.micro_batch_size, sequence_length=cfg.tokens.sequence_length,
        input_pp_rank=trainer.unwrapped_model.input_pp_rank, output_pp_rank=trainer.unwrapped_model.output_pp_rank,
        vocab_size=trainer.model_config.vocab_size, seed=cfg.data_stages[0].data.seed, parallel_context=trainer.parallel_context,
        use_position_ids=not uses_mask,
    )()
