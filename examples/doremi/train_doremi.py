"""Proxy training with DoReMi on synthetic domains (entry point parity: reference examples/doremi/train_doremi.py).

    torchrun --nproc-per-node 2 examples/doremi/train_doremi.py --config-file examples/doremi/config_tiny_doremi.yaml

Without ``doremi.domain_folders`` in the config the data is synthetic: one *learnable* domain (counting sequences) and one
*noise* domain (uniform tokens).  The excess loss concentrates on whichever domain the proxy still lags the reference on, and the
domain weights drift away from uniform, which is what the printed weights show.  Batches come from the domain-weighted sampler of
``dataloader.py``; ``domain_batches`` below is the smallest possible alternative (an endless generator, no datasets).
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from dataloader import get_dataloader  # noqa: E402
from doremi import DoReMiTrainer  # noqa: E402
from utils import get_domain_datasets  # noqa: E402

from nanotron_b200 import distributed as dist  # noqa: E402


def domain_batches(trainer: DoReMiTrainer, seed: int = 0):
    """Infinite micro-batches: every row is drawn from a domain chosen uniformly; ``domain_idxs`` [b] names it."""
    ctx = trainer.parallel_context
    device = ctx.device
    mbs, seq, vocab = trainer.micro_batch_size, trainer.sequence_length, trainer.model_config.vocab_size
    n_domains = trainer.doremi_context.num_domains
    rng = np.random.default_rng(seed * 977 + dist.get_rank(ctx.dp_pg))
    while True:
        doms = rng.integers(0, n_domains, size=mbs)
        rows = []
        for d in doms:
            if d == 0:  # learnable: counting with a small stride
                start, stride = int(rng.integers(0, vocab)), int(rng.integers(1, 4))
                rows.append((start + stride * np.arange(seq + 1)) % vocab)
            else:  # every other domain: noise
                rows.append(rng.integers(0, vocab, size=seq + 1))
        tokens = torch.as_tensor(np.stack(rows), dtype=torch.long, device=device)
        yield {
            "input_ids": tokens[:, :-1].contiguous(), "input_mask": torch.ones(mbs, seq, dtype=torch.bool, device=device),
            "label_ids": tokens[:, 1:].contiguous(), "label_mask": torch.ones(mbs, seq, dtype=torch.bool, device=device),
            "domain_idxs": torch.as_tensor(doms, dtype=torch.long, device=device),
        }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-file", type=str, required=True)
    args = ap.parse_args()
    trainer = DoReMiTrainer(args.config_file)
    datasets = get_domain_datasets(trainer)
    trainer.train({s.name: get_dataloader(trainer, datasets, weights_fn=trainer.sampling_weights) for s in trainer.config.data_stages})


if __name__ == "__main__":
    main()
