"""Writes ``debug_config_tiny_llama.yaml``: the tiny Llama with a layout that fits 4 CPU processes, fp32, verbose logs on every rank
(capability parity: reference examples/contributor-guide/debug_config_tiny_llama.py)."""
import copy
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from config_tiny_llama import config as tiny  # noqa: E402

from nanotron_b200.config import LoggingArgs  # noqa: E402


def build():
    cfg = copy.deepcopy(tiny)
    cfg.general.run = "debug_tiny_llama"
    cfg.general.ignore_sanity_checks = False  # run the invariant checks between the phases of every step
    cfg.parallelism.dp, cfg.parallelism.tp, cfg.parallelism.pp = 2, 2, 1
    cfg.model.dtype = "float32"
    cfg.optimizer.accumulate_grad_in_fp32 = False
    cfg.optimizer.optimizer_factory.torch_adam_is_fused = False
    cfg.logging = LoggingArgs(log_level="debug", log_level_replica="info", iteration_step_info_interval=1)
    cfg.tokens.train_steps = 10
    cfg.checkpoints.checkpoint_interval = 1000
    cfg.checkpoints.save_final_state = False
    cfg.data_stages = cfg.data_stages[:1]
    return cfg


if __name__ == "__main__":
    path = os.path.join(HERE, "debug_config_tiny_llama.yaml")
    build().save_as_yaml(path)
    print(f"wrote {path}")
