"""Configuration of the LlaMoE example and the script that writes ``config_llamoe.yaml``
(capability parity: reference examples/moe/config_llamoe.py).

``LlaMoEConfig`` is a model configuration of its own (a subclass of the Qwen2 one with mixture-of-experts defaults and two extra
knobs), handed to the trainer as ``model_config_class`` together with ``LlaMoEForTraining`` as ``model_class``
(``train_moe.py``).  Where the original example needs the MegaBlocks package, the expert layer here is the framework's own
(``nanotron_b200/nn/moe.py``: router, grouped expert MLP, expert-parallel dispatch / combine, load-balance loss).

    python examples/moe/config_llamoe.py
    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/moe/train_moe.py --config-file examples/moe/config_llamoe.yaml
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nanotron_b200.config import (  # noqa: E402
    AdamWOptimizerArgs, CheckpointsArgs, Config, DataArgs, DatasetStageArgs, GeneralArgs, LoggingArgs, LRSchedulerArgs, ModelArgs, MoEConfig, OptimizerArgs,
    ParallelismArgs, Qwen2Config, RandomInit, TokenizerArgs, TokensArgs,
)


@dataclass
class LlaMoEConfig(Qwen2Config):
    """A Llama-style decoder whose MLPs are mixtures of experts."""

    is_llamoe_config: bool = True  # discriminator in YAML files
    moe_config: Optional[MoEConfig] = field(default_factory=lambda: MoEConfig(num_experts=8, top_k=2, moe_intermediate_size=256, enable_shared_expert=False, router_aux_loss_coef=0.01))
    router_weight_decay: bool = False  # routers are small and sensitive: excluded from weight decay unless asked for
    log_expert_load: bool = True  # keep the per-expert token fractions of the last forward for logging
    # the spelling of the reference example's YAML files (examples/moe/config_llamoe.yaml): when given, they define the experts
    # (every expert as wide as ``intermediate_size``).  Routing here never drops tokens, so the capacity factor has no effect.
    moe_num_experts: Optional[int] = None
    num_experts_per_tok: Optional[int] = None
    moe_capacity_factor: Optional[float] = None

    def __post_init__(self):
        if self.moe_num_experts is not None:
            self.moe_config = MoEConfig(num_experts=self.moe_num_experts, top_k=self.num_experts_per_tok or 1, moe_intermediate_size=self.intermediate_size, enable_shared_expert=False, router_aux_loss_coef=0.01)
        super().__post_init__()


def build(hidden_size=256, layers=4, heads=4, experts=8, top_k=2, expert_size=256, vocab=32000, seq=512, mbs=2, dp=4, ep=4, tp=1, steps=200, dtype="bfloat16", lr=3e-4) -> Config:
    model_config = LlaMoEConfig(
        bos_token_id=1, eos_token_id=2, hidden_size=hidden_size, intermediate_size=4 * hidden_size, max_position_embeddings=seq, num_attention_heads=heads,
        num_hidden_layers=layers, num_key_value_heads=heads, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, vocab_size=vocab,
        moe_config=MoEConfig(num_experts=experts, top_k=top_k, moe_intermediate_size=expert_size, enable_shared_expert=False, router_aux_loss_coef=0.01),
    )
    return Config(
        general=GeneralArgs(project="moe", run="llamoe", seed=42),
        checkpoints=CheckpointsArgs(checkpoints_path="./checkpoints/llamoe", checkpoint_interval=10**6, save_final_state=False),
        parallelism=ParallelismArgs(dp=dp, pp=1, tp=tp, expert_parallel_size=ep, pp_engine="1f1b", tp_mode="REDUCE_SCATTER", tp_linear_async_communication=tp > 1),
        model=ModelArgs(init_method=RandomInit(std=0.02), model_config=model_config, dtype=dtype),
        tokenizer=TokenizerArgs(tokenizer_name_or_path=None),
        optimizer=OptimizerArgs(
            optimizer_factory=AdamWOptimizerArgs(adam_eps=1e-8, adam_beta1=0.9, adam_beta2=0.95, torch_adam_is_fused=dtype == "bfloat16"), zero_stage=0, weight_decay=0.1,
            clip_grad=1.0, accumulate_grad_in_fp32=dtype == "bfloat16",
            learning_rate_scheduler=LRSchedulerArgs(learning_rate=lr, lr_warmup_steps=max(1, steps // 20), lr_warmup_style="linear", lr_decay_style="cosine", min_decay_lr=lr / 10),
        ),
        logging=LoggingArgs(log_level="info", log_level_replica="info", iteration_step_info_interval=10),
        tokens=TokensArgs(sequence_length=seq, train_steps=steps, micro_batch_size=mbs, batch_accumulation_per_replica=1),
        data_stages=[DatasetStageArgs(name="Stable Training Stage", start_training_step=1, data=DataArgs(dataset=None, seed=42, num_loading_workers=0))],
    )


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_llamoe.yaml")
    build().save_as_yaml(out)
    print(f"wrote {out}")
