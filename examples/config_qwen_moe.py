"""Writes ``examples/config_qwen_moe.yaml``: a Qwen2-style mixture-of-experts model (top-4 of 64 experts plus a shared expert, load-balance
loss 0.01) with expert parallelism 8 laid over data parallelism 8 on one node: every GPU holds 8 experts and a full copy of the dense weights.

    python examples/config_qwen_moe.py && torchrun --nproc-per-node 8 run_train.py --config-file examples/config_qwen_moe.yaml

On CUDA the layer runs on the in-tree kernels: router, device-side routing plan, dispatch / combine over NVLink peer memory, grouped tcgen05 GEMMs.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, LRSchedulerArgs, ModelArgs, MoEConfig,
    OptimizerArgs, ParallelismArgs, Qwen2Config, RandomInit, TokenizerArgs, TokensArgs,
)

model_config = Qwen2Config(
    bos_token_id=1, eos_token_id=2, hidden_size=2048, intermediate_size=5632, max_position_embeddings=4096, num_attention_heads=16, num_hidden_layers=24,
    num_key_value_heads=4, rms_norm_eps=1e-06, rope_theta=1000000.0, tie_word_embeddings=False, vocab_size=151936,
    moe_config=MoEConfig(num_experts=64, top_k=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632, enable_shared_expert=True, router_aux_loss_coef=0.01),
)
config = Config(
    general=GeneralArgs(project="moe", run="qwen_moe_%date_%jobid", seed=42),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/qwen-moe", checkpoint_interval=500),
    parallelism=ParallelismArgs(dp=8, pp=1, tp=1, expert_parallel_size=8, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
    model=ModelArgs(init_method=RandomInit(std=0.02), model_config=model_config, dtype="bfloat16"),
    tokenizer=TokenizerArgs(None),
    optimizer=OptimizerArgs(
        zero_stage=0, weight_decay=0.1, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=500, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=3e-5),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-08, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
    ),
    logging=LoggingArgs(iteration_step_info_interval=10),
    tokens=TokensArgs(sequence_length=4096, train_steps=20000, micro_batch_size=2, batch_accumulation_per_replica=4),
    data_stages=[DatasetStageArgs(name="stable", start_training_step=1, data=DataArgs(dataset=None, seed=42))],
)

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_qwen_moe.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
