"""Writes ``config_mamba.yaml`` next to this file (capability parity: reference examples/mamba/create_config_mamba.py).

    python examples/mamba/create_config_mamba.py            # the tiny model of the example
    python examples/mamba/create_config_mamba.py --d-model 768 --layers 24 --out my_mamba.yaml
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from config import MambaConfig, MambaInit, MambaModelArgs, MambaModelConfig  # noqa: E402

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, LRSchedulerArgs, OptimizerArgs, ParallelismArgs, TokenizerArgs, TokensArgs,
)


def build(d_model=64, layers=2, vocab=256, seq=64, mbs=4, steps=40, dp=1, tp=1, pp=1, dtype="float32", lr=3e-3, checkpoints="./checkpoints/mamba") -> MambaConfig:
    model_config = MambaModelConfig(d_model=d_model, num_hidden_layers=layers, vocab_size=vocab, ssm_cfg={"d_state": 8, "d_conv": 4, "expand": 2, "dt_rank": "auto"}, scan_chunk=16)
    return MambaConfig(
        general=GeneralArgs(project="mamba", run="tiny", seed=42),
        checkpoints=CheckpointsArgs(checkpoints_path=checkpoints, checkpoint_interval=10**6, save_final_state=False),
        parallelism=ParallelismArgs(dp=dp, pp=pp, tp=tp, pp_engine="1f1b", tp_mode="ALL_REDUCE", tp_linear_async_communication=False),
        model=MambaModelArgs(model_config=model_config, init_method=MambaInit(initializer_range=0.02), dtype=dtype),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=None),
        optimizer=OptimizerArgs(
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=False), zero_stage=0, weight_decay=0.1, clip_grad=1.0,
            accumulate_grad_in_fp32=False,
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=lr, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=lr / 10),
        ),
        logging=LoggingArgs(log_level="warning", log_level_replica="error", iteration_step_info_interval=10),
        tokens=TokensArgs(sequence_length=seq, train_steps=steps, micro_batch_size=mbs, batch_accumulation_per_replica=1),
        data_stages=[DatasetStageArgs(name="copy task", start_training_step=1, data=DataArgs(dataset=None, seed=42, num_loading_workers=0))],
    )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--d-model", type=int, default=64)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=256)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_mamba.yaml"))
    a = ap.parse_args()
    cfg = build(d_model=a.d_model, layers=a.layers, vocab=a.vocab, seq=a.seq)
    cfg.save_as_yaml(a.out)
    print(f"wrote {a.out}")
