"""Prompt / completion preprocessing for supervised fine-tuning (parity: reference src/nanotron/data/sft_processing.py).

Each example becomes ``input_ids`` (prompt + completion + eos, padded or truncated to ``sequence_length + 1``),
``position_ids`` (0.. inside the example, -1 on padding... padding restarts at 0 so it forms its own document) and a
``label_mask`` that is True only on completion tokens, so the loss ignores the prompt and the padding.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np


def process_sft(examples: Dict[str, List[str]], tokenizer, sequence_length: int, prompt_column: str = "prompt", completion_column: str = "completion") -> Dict[str, List[np.ndarray]]:
    out = {"input_ids": [], "position_ids": [], "label_mask": []}
    eos = tokenizer.eos_token_id if tokenizer.eos_token_id is not None else 0
    pad = tokenizer.pad_token_id if getattr(tokenizer, "pad_token_id", None) is not None else eos
    for prompt, completion in zip(examples[prompt_column], examples[completion_column]):
        p = tokenizer(prompt, add_special_tokens=False)["input_ids"]
        c = tokenizer(completion, add_special_tokens=False)["input_ids"] + [eos]
        ids = (p + c)[: sequence_length + 1]
        n_prompt = min(len(p), len(ids))
        n = len(ids)
        mask = np.zeros(sequence_length + 1, dtype=np.bool_)
        mask[n_prompt:n] = True
        padded = np.full(sequence_length + 1, pad, dtype=np.int64)
        padded[:n] = ids
        pos = np.zeros(sequence_length + 1, dtype=np.int64)
        pos[:n] = np.arange(n)
        pos[n:] = np.arange(sequence_length + 1 - n)  # padding is a separate "document" starting at 0
        out["input_ids"].append(padded)
        out["position_ids"].append(pos)
        out["label_mask"].append(mask)
    return out


def prepare_sft_dataset(raw_dataset, tokenizer, trainer_sequence_length: int, debug_max_samples=None, num_proc: int = 1):
    if debug_max_samples is not None:
        raw_dataset = raw_dataset.select(range(min(debug_max_samples, len(raw_dataset))))
    cols = raw_dataset.column_names
    prompt_col = "prompt" if "prompt" in cols else cols[0]
    completion_col = "completion" if "completion" in cols else cols[1]
    return raw_dataset.map(
        lambda ex: process_sft(ex, tokenizer, trainer_sequence_length, prompt_col, completion_col),
        batched=True, remove_columns=cols, num_proc=num_proc, desc="Tokenising prompt/completion pairs",
    )
