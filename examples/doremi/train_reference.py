"""Training on a fixed mixture of the domains: the small reference model of a DoReMi run, or the final large model on the tuned
weights (entry point parity: reference examples/doremi/train_reference.py).

    torchrun --nproc-per-node 2 examples/doremi/train_reference.py --config-file examples/doremi/config_tiny_doremi.yaml

The mixture is ``doremi.domain_weights`` of the config; ``--token-count-weights`` replaces it by the domains' shares of the data
(no domain runs out before the others); without either it is uniform.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from dataloader import domain_weights_from_token_count, get_dataloader  # noqa: E402
from doremi import DoReMiConfig, ReferenceTrainer  # noqa: E402
from utils import get_domain_datasets, print_array_for_human  # noqa: E402

from nanotron_b200 import logging  # noqa: E402
from nanotron_b200.config import get_config_from_file  # noqa: E402
from nanotron_b200.logging import log_rank  # noqa: E402

logger = logging.get_logger(__name__)


def build(config_file: str, token_count_weights: bool = False) -> ReferenceTrainer:
    weights = None
    if token_count_weights:
        # the datasets are needed before the trainer exists: sizes only, so a bare object with the fields the loader reads is enough
        config = get_config_from_file(config_file, config_class=DoReMiConfig)

        class _Shape:
            pass

        shape = _Shape()
        shape.config, shape.sequence_length, shape.model_config = config, config.tokens.sequence_length, config.model.model_config
        weights = domain_weights_from_token_count(get_domain_datasets(shape))
    return ReferenceTrainer(config_file, domain_weights=weights)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-file", type=str, required=True)
    ap.add_argument("--token-count-weights", action="store_true")
    args = ap.parse_args()
    trainer = build(args.config_file, args.token_count_weights)
    log_rank(f"[DoReMi] training on the mixture {print_array_for_human(trainer.doremi_context.domain_weights)}", logger=logger, level=logging.INFO, rank=0)
    datasets = get_domain_datasets(trainer)
    trainer.train({s.name: get_dataloader(trainer, datasets, weights_fn=trainer.sampling_weights) for s in trainer.config.data_stages})


if __name__ == "__main__":
    main()
