"""Writes ``examples/doremi/config_tiny_doremi.yaml``: a tiny Llama proxy with a ``doremi`` section (two synthetic domains)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from doremi import DoReMiArgs, DoReMiConfig  # noqa: E402

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, DataArgs, DatasetStageArgs, GeneralArgs, LlamaConfig, LoggingArgs, LRSchedulerArgs, ModelArgs, OptimizerArgs,
    ParallelismArgs, RandomInit, TokenizerArgs, TokensArgs,
)

config = DoReMiConfig(
    general=GeneralArgs(project="doremi", run="tiny_proxy", seed=42),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/doremi", checkpoint_interval=1000),
    parallelism=ParallelismArgs(dp=2, pp=1, tp=1),
    model=ModelArgs(init_method=RandomInit(std=0.025), dtype="float32", model_config=LlamaConfig(
        hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, vocab_size=128, max_position_embeddings=64, rms_norm_eps=1e-5)),
    tokenizer=TokenizerArgs(None),
    optimizer=OptimizerArgs(
        zero_stage=0, weight_decay=0.01, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-3, lr_warmup_steps=2, lr_decay_style="cosine", min_decay_lr=3e-4),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=False),
    ),
    logging=LoggingArgs(iteration_step_info_interval=5),
    tokens=TokensArgs(sequence_length=64, train_steps=60, micro_batch_size=4, batch_accumulation_per_replica=1),
    data_stages=[DatasetStageArgs(name="proxy", start_training_step=1, data=DataArgs(dataset=None, seed=7))],
    doremi=DoReMiArgs(domain_names=["counting", "noise"], step_size=1.0, smoothing_param=1e-3),
)

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_tiny_doremi.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
