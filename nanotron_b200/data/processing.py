"""Tokenise-and-pack preprocessing for HuggingFace text datasets (parity: reference src/nanotron/data/processing.py)."""
from __future__ import annotations

from typing import Dict, List

import numpy as np


def group_texts(token_lists: List[List[int]], sequence_length: int) -> Dict[str, List[np.ndarray]]:
    """Concatenate all tokens and cut them into windows of ``sequence_length + 1`` that overlap by one token, so that
    after the collator's shift every window yields ``sequence_length`` (input, label) pairs.  The tail is dropped."""
    concatenated = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists]) if token_lists else np.zeros(0, dtype=np.int64)
    total = len(concatenated)
    if total >= sequence_length + 1:
        total = ((total - 1) // sequence_length) * sequence_length + 1
    else:
        total = 0
    return {"input_ids": [concatenated[i : i + sequence_length + 1] for i in range(0, total - (sequence_length + 1) + 1, sequence_length)]}


def clm_process(raw_dataset, tokenizer, text_column_name: str, dataset_processing_num_proc_per_process: int, dataset_overwrite_cache: bool, sequence_length: int):
    """``datasets.Dataset`` of text -> dataset of packed ``input_ids`` windows (length ``sequence_length + 1``)."""

    def _tokenize_and_group(texts: List[str]) -> Dict[str, List[np.ndarray]]:
        # the plain call works with every transformers version (``batch_encode_plus`` is gone from the 5.x tokenizers)
        tokenized = tokenizer(list(texts), return_attention_mask=False, return_token_type_ids=False)
        return group_texts(tokenized["input_ids"], sequence_length)

    from datasets import Features, Sequence, Value

    return raw_dataset.map(
        _tokenize_and_group,
        input_columns=text_column_name,
        remove_columns=raw_dataset.column_names,
        features=Features({"input_ids": Sequence(feature=Value(dtype="int64"), length=sequence_length + 1)}),
        batched=True,
        num_proc=dataset_processing_num_proc_per_process,
        load_from_cache_file=not dataset_overwrite_cache,
        desc=f"Grouping texts in chunks of {sequence_length + 1}",
    )


def get_datasets(hf_dataset_or_datasets, hf_dataset_config_name, splits="train"):
    """Load one or several HuggingFace datasets / splits and concatenate them per split."""
    from datasets import DatasetDict, concatenate_datasets, load_dataset

    if isinstance(splits, str):
        splits = [splits]
    if isinstance(hf_dataset_or_datasets, dict):
        raise ValueError("dict of datasets is not supported; use a list or a single name")
    names = [hf_dataset_or_datasets] if isinstance(hf_dataset_or_datasets, str) else list(hf_dataset_or_datasets)
    out = DatasetDict()
    for split in splits:
        parts = [load_dataset(n, hf_dataset_config_name, split=split) for n in names]
        out[split] = parts[0] if len(parts) == 1 else concatenate_datasets(parts)
    return out
