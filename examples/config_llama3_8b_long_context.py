"""Writes ``examples/config_llama3_8b_long_context.yaml``: Llama-3-8B shapes (through the Qwen2 model family, which carries the packed /
context-parallel attention path) at sequence length 65536 with context parallelism 8: every GPU holds two zig-zag chunks of 4096 tokens of each
sequence.  ``_attn_implementation: ring_fused`` keeps keys and values on their owners and lets the attention kernels fetch / reduce them over NVLink;
``llama3_ring_attention`` is the NCCL all-gather + library-attention path.

    python examples/config_llama3_8b_long_context.py && torchrun --nproc-per-node 8 run_train.py --config-file examples/config_llama3_8b_long_context.yaml
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, LRSchedulerArgs, ModelArgs, OptimizerArgs,
    ParallelismArgs, Qwen2Config, RandomInit, TokenizerArgs, TokensArgs,
)

model_config = Qwen2Config(
    bos_token_id=128000, eos_token_id=128001, hidden_size=4096, intermediate_size=14336, max_position_embeddings=65536, num_attention_heads=32,
    num_hidden_layers=32, num_key_value_heads=8, rms_norm_eps=1e-05, rope_theta=500000.0, tie_word_embeddings=False, vocab_size=128256,
    attention_bias=False, _attn_implementation="llama3_ring_attention", ring_attn_heads_k_stride=1,
)
config = Config(
    general=GeneralArgs(project="llama3", run="8b_64k_%date_%jobid", seed=42),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/llama3-8b-64k", checkpoint_interval=200),
    parallelism=ParallelismArgs(dp=1, pp=1, tp=1, context_parallel_size=8, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True, recompute_layer=True),
    model=ModelArgs(init_method=RandomInit(std=0.02), model_config=model_config, dtype="bfloat16"),
    tokenizer=TokenizerArgs(None),
    optimizer=OptimizerArgs(
        zero_stage=0, weight_decay=0.1, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=1e-5, lr_warmup_steps=20, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=1e-6),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-08, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
    ),
    logging=LoggingArgs(iteration_step_info_interval=1),
    tokens=TokensArgs(sequence_length=65536, train_steps=1000, micro_batch_size=1, batch_accumulation_per_replica=8),
    data_stages=[DatasetStageArgs(name="stable", start_training_step=1, data=DataArgs(dataset=None, seed=42))],
)

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_llama3_8b_long_context.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
