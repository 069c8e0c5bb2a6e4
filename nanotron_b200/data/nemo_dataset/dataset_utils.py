"""Helpers shared by the Megatron-style datasets (capability parity: reference
src/nanotron/data/nemo_dataset/dataset_utils.py:25-105)."""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple, Union


def compile_helper():
    """Build the C++ index helpers in place (the reference runs ``make`` in the package directory)."""
    from nanotron_b200.ops.build import build_data_helpers

    build_data_helpers()


def get_datasets_weights_and_num_samples(data_prefix: Sequence[Union[str, float]], num_samples: Union[int, List[int]]) -> Tuple[List[str], List[float], List]:
    """``data_prefix`` alternates weights and path prefixes: [w0, p0, w1, p1, ...].  Weights are normalised; every dataset is
    asked for 0.5 % more samples than its share so that blending never runs dry."""
    assert len(data_prefix) % 2 == 0, "expected alternating weights and prefixes"
    n = len(data_prefix) // 2
    weights = [float(data_prefix[2 * i]) for i in range(n)]
    prefixes = [str(data_prefix[2 * i + 1]).strip() for i in range(n)]
    total = sum(weights)
    assert total > 0.0
    weights = [w / total for w in weights]
    if isinstance(num_samples, (list, tuple)):
        per_dataset = [[int(math.ceil(v * w * 1.005)) for v in num_samples] for w in weights]
    else:
        per_dataset = [int(math.ceil(num_samples * w * 1.005)) for w in weights]
    return prefixes, weights, per_dataset


def get_train_valid_test_split_(splits_string: str, size: int) -> List[int]:
    """'949,50,1' (or '98/1/1') -> the four boundaries [0, a, b, size] of the train / valid / test document ranges."""
    sep = "," if "," in splits_string else ("/" if "/" in splits_string else None)
    parts = [float(s) for s in splits_string.split(sep)] if sep else [float(splits_string)]
    parts = (parts + [0.0, 0.0, 0.0])[:3]
    total = sum(parts)
    assert total > 0.0
    fractions = [p / total for p in parts]
    index = [0]
    for f in fractions:
        index.append(index[-1] + int(round(f * float(size))))
    diff = index[-1] - size
    index = [index[0]] + [v - diff for v in index[1:]]
    assert len(index) == 4 and index[-1] == size
    return index
