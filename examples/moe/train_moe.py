"""Trains the LlaMoE example (capability parity: reference examples/moe/train_moe.py): the stock trainer with the example's
model configuration class and model class.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/moe/train_moe.py --config-file examples/moe/config_llamoe.yaml
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from config_llamoe import LlaMoEConfig  # noqa: E402
from llamoe import LlaMoEForTraining  # noqa: E402

from nanotron_b200.trainer import DistributedTrainer  # noqa: E402


def make_trainer(config_or_file) -> DistributedTrainer:
    return DistributedTrainer(config_or_file, model_config_class=LlaMoEConfig, model_class=LlaMoEForTraining)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-file", type=str, required=True)
    args = ap.parse_args()
    trainer = make_trainer(args.config_file)
    from run_train import get_dataloader

    trainer.train(get_dataloader(trainer))
    report = trainer.unwrapped_model.expert_load_report()
    if report:
        print("largest expert share per router in the last forward:", {k: round(v, 3) for k, v in report.items()})
