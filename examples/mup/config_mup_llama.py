"""Spectral µTransfer (µP) against the standard parametrisation on a Llama of configurable width
(capability parity: reference examples/mup/configs/{mup,sp}_350m_llama_config.yaml and its README).

    python examples/mup/config_mup_llama.py                    # writes mup_350m_llama_config.yaml and sp_350m_llama_config.yaml
    python examples/mup/config_mup_llama.py --hidden-size 256 --layers 4 --out-dir /tmp/mup_small

The only difference between the two files is the ``init_method`` of the model section:

    init_method:                      init_method:
      std: 0.025          ->            use_mup: true

With ``use_mup`` the framework picks each matrix's initial standard deviation and learning-rate multiplier from its fan-in / fan-out
(``nanotron_b200/scaling/parametrization.py``: spectral condition, std ~ sqrt(fan_out / fan_in) / sqrt(fan_in), learning rate ~ fan_out / fan_in),
so a learning rate tuned on a narrow model carries over to wider ones.  ``sweep_widths`` below builds the configs of such a width sweep.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LlamaConfig, LoggingArgs, LRSchedulerArgs, ModelArgs, OptimizerArgs,
    ParallelismArgs, RandomInit, SpectralMupInit, TokenizerArgs, TokensArgs,
)


def build(use_mup: bool, hidden_size: int = 1024, layers: int = 24, heads: int = 16, vocab: int = 49152, seq: int = 2048, mbs: int = 4, acc: int = 16, dp: int = 8,
          steps: int = 15000, lr: float = 1e-3, dtype: str = "bfloat16") -> Config:
    model_config = LlamaConfig(
        bos_token_id=1, eos_token_id=2, hidden_act="silu", hidden_size=hidden_size, initializer_range=0.02, intermediate_size=4 * hidden_size, max_position_embeddings=seq,
        num_attention_heads=heads, num_hidden_layers=layers, num_key_value_heads=heads, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, vocab_size=vocab,
    )
    name = "mup" if use_mup else "sp"
    return Config(
        general=GeneralArgs(project="mup_transfer", run=f"{name}_h{hidden_size}_l{layers}", seed=42),
        checkpoints=CheckpointsArgs(checkpoints_path=f"./checkpoints/{name}_h{hidden_size}", checkpoint_interval=5000),
        parallelism=ParallelismArgs(dp=dp, pp=1, tp=1, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
        model=ModelArgs(init_method=SpectralMupInit(use_mup=True) if use_mup else RandomInit(std=0.025), model_config=model_config, dtype=dtype),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=None),
        optimizer=OptimizerArgs(
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True), zero_stage=0, weight_decay=0.1, clip_grad=1.0,
            accumulate_grad_in_fp32=dtype == "bfloat16",
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=lr, lr_warmup_steps=max(1, steps // 100), lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=lr / 10),
        ),
        logging=LoggingArgs(log_level="info", log_level_replica="info", iteration_step_info_interval=10),
        tokens=TokensArgs(sequence_length=seq, train_steps=steps, micro_batch_size=mbs, batch_accumulation_per_replica=acc),
        data_stages=[DatasetStageArgs(name="Stable Training Stage", start_training_step=1, data=DataArgs(dataset=None, seed=42, num_loading_workers=1))],
    )


def sweep_widths(widths=(256, 512, 1024, 2048), **kw):
    """One µP config per width, everything else equal: the learning rate found at the narrowest is meant to be reused as is."""
    return {w: build(use_mup=True, hidden_size=w, heads=max(1, w // 64), **kw) for w in widths}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden-size", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--out-dir", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs"))
    a = ap.parse_args()
    os.makedirs(a.out_dir, exist_ok=True)
    for use_mup in (True, False):
        path = os.path.join(a.out_dir, f"{'mup' if use_mup else 'sp'}_350m_llama_config.yaml")
        build(use_mup, hidden_size=a.hidden_size, layers=a.layers, heads=max(1, a.hidden_size // 64)).save_as_yaml(path)
        print(f"wrote {path}")
