"""Benchmark configuration of a Llama-2-7B-shaped model (capability parity: reference examples/bench_llama_7b.py).

    python examples/bench_llama_7b.py                                   # writes examples/config_bench_llama_7b.yaml
    NANOTRON_BENCHMARK=1 torchrun --nproc-per-node 8 --master-addr 127.0.0.1 run_train.py --config-file examples/config_bench_llama_7b.yaml

With ``NANOTRON_BENCHMARK=1`` the trainer reports throughput (tokens/s, tokens/s/GPU, model TFLOP/s per GPU, memory) on the fourth step,
appends the row to ``general.benchmark_csv_path`` and stops.  Data is the dummy generator (random tokens): nothing has to be downloaded.
``bench.py`` at the repository root is the stricter harness (device timing over several steps, clock sampling, one JSON line).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LlamaConfig, LoggingArgs, LRSchedulerArgs, ModelArgs, OptimizerArgs,
    ParallelismArgs, RandomInit, TokenizerArgs, TokensArgs,
)
from nanotron_b200.logging import human_format  # noqa: E402

model_config = LlamaConfig(
    bos_token_id=1, eos_token_id=2, hidden_act="silu", hidden_size=4096, initializer_range=0.02, intermediate_size=11008, max_position_embeddings=8192,
    num_attention_heads=32, num_hidden_layers=32, num_key_value_heads=32, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, vocab_size=32000,
)
num_params = model_config.vocab_size * model_config.hidden_size * 2 + model_config.num_hidden_layers * (
    3 * model_config.hidden_size * model_config.intermediate_size + 4 * model_config.hidden_size * model_config.hidden_size
)

config = Config(
    general=GeneralArgs(project="bench", run="llama_7b", seed=42, benchmark_csv_path="bench_llama_7b.csv"),
    checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/bench_llama_7b", checkpoint_interval=10**6, save_final_state=False),
    parallelism=ParallelismArgs(dp=2, pp=1, tp=4, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=True),
    model=ModelArgs(init_method=RandomInit(std=0.025), model_config=model_config),
    tokenizer=TokenizerArgs(tokenizer_name_or_path=None),
    optimizer=OptimizerArgs(
        zero_stage=1, weight_decay=0.01, clip_grad=1.0, accumulate_grad_in_fp32=True,
        learning_rate_scheduler=LRSchedulerArgs(learning_rate=3e-4, lr_warmup_steps=2, lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=1e-5),
        optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=True),
    ),
    logging=LoggingArgs(iteration_step_info_interval=1),
    tokens=TokensArgs(sequence_length=8192, train_steps=5, micro_batch_size=1, batch_accumulation_per_replica=8),
    data_stages=[DatasetStageArgs(name="bench", start_training_step=1, data=DataArgs(dataset=None, seed=42, num_loading_workers=0))],
)

if __name__ == "__main__":
    print(f"Model has {human_format(num_params)} parameters")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_bench_llama_7b.yaml")
    config.save_as_yaml(path)
    print(f"wrote {path}")
