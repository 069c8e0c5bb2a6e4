"""Writes ``examples/config_llama3_8b.yaml``: Llama-3-8B on one 8 x B200 node, data parallel 8 with ZeRO-1 (the layout `bench.py` measures).

    python examples/config_llama3_8b.py && torchrun --nproc-per-node 8 run_train.py --config-file examples/config_llama3_8b.yaml

Replace ``dataset=None`` (random tokens) by a ``NanosetDatasetsArgs`` / ``PretrainDatasetsArgs`` block for real data.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LlamaConfig, LoggingArgs, LRSchedulerArgs,
    ModelArgs, OptimizerArgs, ParallelismArgs, RandomInit, TokenizerArgs, TokensArgs,
)

model_config = LlamaConfig(
    bos_token_id=128000, eos_token_id=128001, hidden_act="silu", hidden_size=4096, initializer_range=0.02, intermediate_size=14336, max_position_embeddings=4096,
    num_attention_heads=32, num_hidden_layers=32, num_key_value_heads=8, rms_norm_eps=1e-05, rope_theta=500000.0, tie_word_embeddings=False, vocab_size=128256,
)
config = Config(
    general=GeneralArgs(project="llama3", run="8b_%date_%jobid", seed=42),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/llama3-8b", checkpoint_interval=500),
    parallelism=ParallelismArgs(dp=8, pp=1, tp=1, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
    model=ModelArgs(init_method=RandomInit(std=0.02), model_config=model_config, dtype="bfloat16"),
    tokenizer=TokenizerArgs(None),
    optimizer=OptimizerArgs(
        zero_stage=1, weight_decay=0.1, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2000, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=3e-5),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-08, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
    ),
    logging=LoggingArgs(iteration_step_info_interval=10),
    tokens=TokensArgs(sequence_length=4096, train_steps=100000, micro_batch_size=1, batch_accumulation_per_replica=8),
    data_stages=[DatasetStageArgs(name="stable", start_training_step=1, data=DataArgs(dataset=None, seed=42))],
)

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_llama3_8b.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
