"""The domains of the DoReMi example: folders of tokenised files when the config names them, synthetic ones otherwise
(capability parity: reference examples/doremi/doremi/dataloader.py ``get_datasets`` and examples/doremi/utils.py)."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
from torch.utils.data import Dataset


class SyntheticDomain(Dataset):
    """``num_samples`` sequences of ``length`` tokens; item ``i`` is a pure function of (kind, seed, i).

    ``counting``: (start + i * stride) mod vocab with a small stride -- learnable down to almost zero loss;
    ``repeat``:   a random block of 4 tokens repeated -- learnable after the first block;
    ``noise``:    uniform tokens -- nothing to learn, the loss stays at log(vocab)."""

    KINDS = ("counting", "repeat", "noise")

    def __init__(self, kind: str, num_samples: int, length: int, vocab_size: int, seed: int = 0):
        assert kind in self.KINDS, f"unknown synthetic domain {kind!r}"
        self.kind, self.num_samples, self.length, self.vocab_size, self.seed = kind, num_samples, length, vocab_size, seed

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, i: int):
        rng = np.random.default_rng([self.seed, self.KINDS.index(self.kind), int(i)])
        if self.kind == "counting":
            start, stride = int(rng.integers(0, self.vocab_size)), int(rng.integers(1, 4))
            ids = (start + stride * np.arange(self.length, dtype=np.int64)) % self.vocab_size
        elif self.kind == "repeat":
            block = rng.integers(0, self.vocab_size, size=4)
            ids = np.tile(block, self.length // 4 + 1)[: self.length].astype(np.int64)
        else:
            ids = rng.integers(0, self.vocab_size, size=self.length).astype(np.int64)
        return {"input_ids": ids}


def get_domain_datasets(trainer) -> List[Dataset]:
    """One dataset per entry of ``doremi.domain_names``; every item holds ``sequence_length + 1`` token ids."""
    args = trainer.config.doremi
    seq = trainer.sequence_length
    if args.domain_folders is not None:
        from nanotron_b200.data.nanoset import TokenFolderDataset

        return [TokenFolderDataset(folder, seq, args.token_size, shuffle=False, seed=trainer.config.data_stages[0].data.seed, return_positions=False) for folder in args.domain_folders]
    kinds = [name if name in SyntheticDomain.KINDS else "noise" for name in args.domain_names]
    return [SyntheticDomain(kind, args.samples_per_synthetic_domain, seq + 1, trainer.model_config.vocab_size, seed=trainer.config.data_stages[0].data.seed) for kind in kinds]


def print_array_for_human(values: Sequence[float], precision: int = 5) -> str:
    return "[" + ", ".join(f"{float(v):.{precision}f}" for v in values) + "]"
