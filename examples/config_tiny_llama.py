"""Writes ``examples/config_tiny_llama.yaml``: a tiny Llama on dummy data, dp2 x tp2 x pp2 (8 processes)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LlamaConfig, LoggingArgs, LRSchedulerArgs,
    ModelArgs, OptimizerArgs, ParallelismArgs, RandomInit, TokenizerArgs, TokensArgs,
)

model_config = LlamaConfig(
    bos_token_id=1, eos_token_id=2, hidden_act="silu", hidden_size=16, initializer_range=0.02, intermediate_size=64, max_position_embeddings=256,
    num_attention_heads=4, num_hidden_layers=2, num_key_value_heads=4, rms_norm_eps=1e-05, tie_word_embeddings=True, vocab_size=256,
)
config = Config(
    general=GeneralArgs(project="debug", run="tiny_llama_%date_%jobid", seed=42),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints", checkpoint_interval=10),
    parallelism=ParallelismArgs(dp=2, pp=2, tp=2, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
    model=ModelArgs(init_method=RandomInit(std=0.025), model_config=model_config),
    tokenizer=TokenizerArgs(None),
    optimizer=OptimizerArgs(
        zero_stage=1, weight_decay=0.01, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=1e-5),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-08, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
    ),
    logging=LoggingArgs(),
    tokens=TokensArgs(sequence_length=256, train_steps=15, micro_batch_size=2, batch_accumulation_per_replica=1),
    data_stages=[
        DatasetStageArgs(name="Stable Training Stage", start_training_step=1, data=DataArgs(dataset=None, seed=42)),
        DatasetStageArgs(name="Annealing Phase", start_training_step=10, data=DataArgs(dataset=None, seed=43)),
    ],
)

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_tiny_llama.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
