"""Small numeric helpers for dataset blending (parity: reference src/nanotron/data/utils.py)."""
from typing import List

import numpy as np


def normalize(weights: List[float]) -> np.ndarray:
    w = np.array(weights, dtype=np.float64)
    return w / np.sum(w)


def count_dataset_indexes(dataset_idx: np.ndarray, n_datasets: int) -> np.ndarray:
    return np.bincount(np.asarray(dataset_idx, dtype=np.int64), minlength=n_datasets)
