"""Weighted mixtures of datasets (capability parity: reference src/nanotron/data/nemo_dataset/blendable_dataset.py:43-292).

``BlendableDataset`` materialises, for every index of the blend, which dataset it draws from and which of that dataset's samples
(the greedy "largest deficit first" interleave of the C++ helper ``build_blending_indices``).  ``MemoryEfficientBlendableDataset``
derives the same kind of mapping arithmetically from a small table of ``weight_bins`` slots instead of storing it.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.logging import log_rank

logger = logging.get_logger(__name__)


@dataclass
class BlendedSubsetSplitLog:
    blended_total_num_samples: int
    blended_per_subset_samples: List[int]
    blended_subset: List = field(default_factory=list)


def _blend_numpy(weights: np.ndarray, size: int):
    """Numpy statement of the interleave: at every step take the dataset whose share so far lags its weight the most."""
    n = len(weights)
    index = np.zeros(size, dtype=np.int16)
    sample_index = np.zeros(size, dtype=np.int64)
    counts = np.zeros(n, dtype=np.int64)
    for i in range(size):
        denom = max(float(i), 1.0)
        errors = weights * denom - counts
        k = int(np.argmax(errors))
        index[i], sample_index[i] = k, counts[k]
        counts[k] += 1
    return index, sample_index, counts


class BlendableDataset(torch.utils.data.Dataset):
    def __init__(self, datasets: List, weights: List[float], size: int, parallel_context=None, seed: int = 0, consumed_samples: int = 0,
                 dataset_name: Optional[str] = None, consumed_tokens_per_dataset_folder: Optional[Dict[str, int]] = None,
                 offsets_in_samples: Optional[Dict[str, int]] = None):
        self.datasets = datasets
        n = len(datasets)
        assert n == len(weights) and n < 32767
        self.size = size
        self.random_seed = seed
        w = np.asarray(weights, dtype=np.float64)
        assert w.sum() > 0.0
        w = w / w.sum()
        t0 = time.time()
        self.dataset_index = np.zeros(size, dtype=np.int16)
        self.dataset_sample_index = np.zeros(size, dtype=np.int64)
        self.dataset_num_samples = np.zeros(n, dtype=np.int64)
        try:
            from nanotron_b200.data.nemo_dataset import helpers

            helpers.build_blending_indices(self.dataset_index, self.dataset_sample_index, self.dataset_num_samples, w, n, size, False)
        except (ImportError, OSError):
            self.dataset_index, self.dataset_sample_index, self.dataset_num_samples = _blend_numpy(w, size)
        log_rank(f"> built blendable dataset indices in {time.time() - t0:.2f} s", logger=logger, level=logging.INFO, rank=0)
        self.subset_log = BlendedSubsetSplitLog(blended_total_num_samples=size, blended_per_subset_samples=self.dataset_num_samples.tolist(),
                                                blended_subset=[getattr(d, "subset_log", None) for d in datasets])
        # per-dataset consumption bookkeeping (tokens seen in this stage; sample offsets carried over from earlier stages)
        self.consumed_tokens = {i: 0 for i in range(n)}
        self.offsets_in_samples = {i: 0 for i in range(n)}
        for table, given in ((self.consumed_tokens, consumed_tokens_per_dataset_folder), (self.offsets_in_samples, offsets_in_samples)):
            if given:
                for i, d in enumerate(datasets):
                    folder = getattr(d, "folder_path", None)
                    if folder in given:
                        table[i] = given[folder]
        self.sequence_length = None

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, idx):
        k = int(self.dataset_index[idx])
        return self.datasets[k][int(self.dataset_sample_index[idx]) + self.offsets_in_samples[k]]

    def update_consumption_metrics(self, start_idx: int, end_idx: int, sequence_length: int):
        """Account the samples [start_idx, end_idx) of the blend (one global batch) to their datasets."""
        if self.sequence_length is None:
            self.sequence_length = sequence_length
        which, counts = np.unique(self.dataset_index[start_idx:end_idx], return_counts=True)
        for k, c in zip(which, counts):
            self.consumed_tokens[int(k)] += int(c * sequence_length)

    def get_consumption_stats(self) -> Dict[str, Dict[str, int]]:
        return {getattr(d, "folder_path", str(i)): {"tokens": self.consumed_tokens[i]} for i, d in enumerate(self.datasets)}


class MemoryEfficientBlendableDataset(torch.utils.data.Dataset):
    """Index i falls in slot ``i % weight_bins``; slots are handed to the datasets in proportion to their weights, and the
    j-th visit of a slot reads the next unread sample of its dataset (modulo the dataset's length)."""

    def __init__(self, datasets, weights, size: int, weight_bins: int = 100):
        self.datasets = datasets
        n = len(datasets)
        assert n == len(weights)
        weight_bins = min(weight_bins, size)
        self.size, self.weight_bins = size, weight_bins
        w = np.asarray(weights, dtype=np.float64)
        assert (w > 0.0).all()
        self.weights = w / w.sum()
        slots, bias = [], []
        for i, wi in enumerate(self.weights):
            k = int(wi * weight_bins)
            slots += [i] * k
            bias += list(range(k))
        rest = weight_bins - len(slots)  # rounding remainder goes to the last dataset
        slots += [n - 1] * rest
        bias += list(range(bias[-1], bias[-1] + rest))
        self.ds_index = np.asarray(slots, dtype=np.uint32)
        self.ds_bias = np.asarray(bias, dtype=np.uint32)
        self.ds_index_size = np.asarray([(self.ds_index == i).sum() for i in range(n)], dtype=np.uint32)
        assert (self.ds_index_size > 0).all(), f"a dataset got no slot: raise weight_bins or its weight ({self.ds_index_size})"
        self.ds_size = np.asarray([len(d) for d in datasets], dtype=np.uint32)

    def get_ds_sample_idx(self, idx: int):
        slot = idx % self.weight_bins
        k = int(self.ds_index[slot])
        return k, int((int(self.ds_bias[slot]) + (idx // self.weight_bins) * int(self.ds_index_size[k])) % int(self.ds_size[k]))

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, idx):
        k, j = self.get_ds_sample_idx(idx)
        return self.datasets[k][j]
