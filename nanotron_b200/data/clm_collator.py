"""Batch collators for causal language modelling (parity: reference src/nanotron/data/clm_collator.py).

All collators take examples of ``sequence_length + 1`` tokens, shift by one to build labels, hand real tensors only to
the pipeline stages that need them (``TensorPointer`` elsewhere) and cut the sequence for context parallelism.  The
context-parallel cut is zig-zag here (balanced causal work); position ids stay global.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Union

import numpy as np
import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.parallel.context import ParallelContext
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer


def _cp_cut(x: np.ndarray, cp_rank: int, cp_size: int, zigzag: bool) -> np.ndarray:
    if cp_size == 1:
        return x
    n = x.shape[1]
    if zigzag:
        assert n % (2 * cp_size) == 0, f"sequence length {n} must be divisible by 2*cp={2 * cp_size}"
        c = n // (2 * cp_size)
        a, b = cp_rank, 2 * cp_size - 1 - cp_rank
        return np.concatenate([x[:, a * c : (a + 1) * c], x[:, b * c : (b + 1) * c]], axis=1)
    per = n // cp_size
    return x[:, cp_rank * per : (cp_rank + 1) * per]


@dataclasses.dataclass
class DataCollatorForCLM:
    """Outputs ``input_ids, input_mask, label_ids, label_mask`` (Llama-style models)."""

    sequence_length: int
    input_pp_rank: int
    output_pp_rank: int
    parallel_context: ParallelContext
    use_numpy: bool = True
    cp_zigzag: bool = True

    def __call__(self, examples: List[Dict[str, np.ndarray]]) -> Dict[str, Union[np.ndarray, TensorPointer]]:
        ctx = self.parallel_context
        pp_rank = dist.get_rank(ctx.pp_pg)
        result: Dict[str, Union[np.ndarray, TensorPointer]] = {
            "input_ids": TensorPointer(group_rank=self.input_pp_rank),
            "input_mask": TensorPointer(group_rank=self.input_pp_rank),
            "label_ids": TensorPointer(group_rank=self.output_pp_rank),
            "label_mask": TensorPointer(group_rank=self.output_pp_rank),
        }
        if pp_rank not in (self.input_pp_rank, self.output_pp_rank):
            assert all(len(e) == 0 for e in examples)
            return result
        input_ids = np.vstack([np.asarray(e["input_ids"]) for e in examples])
        batch, length = input_ids.shape
        assert length == self.sequence_length + 1, f"Samples should be of length {self.sequence_length + 1} (seq_len+1), but got {length}"
        cp_rank, cp_size = dist.get_rank(ctx.cp_pg), ctx.context_parallel_size
        if pp_rank == self.input_pp_rank:
            result["input_ids"] = _cp_cut(input_ids[:, :-1], cp_rank, cp_size, self.cp_zigzag)
            result["input_mask"] = np.ones(result["input_ids"].shape, dtype=np.bool_)
        if pp_rank == self.output_pp_rank:
            mask = np.ones((batch, self.sequence_length), dtype=np.bool_)
            if "positions" in examples[0]:
                positions = np.vstack([np.asarray(e["positions"]) for e in examples])[:, 1:]
                mask &= positions != 0  # do not predict the first token of the next document
            result["label_ids"] = _cp_cut(input_ids[:, 1:], cp_rank, cp_size, self.cp_zigzag)
            result["label_mask"] = _cp_cut(mask, cp_rank, cp_size, self.cp_zigzag)
        if not self.use_numpy:
            result = {k: (torch.from_numpy(np.ascontiguousarray(v)) if isinstance(v, np.ndarray) else v) for k, v in result.items()}
        return result


@dataclasses.dataclass
class DataCollatorForCLMWithPositionIds:
    """Outputs ``input_ids, position_ids, label_ids, label_mask`` (Qwen2-style packed documents: a position id of 0
    starts a document).  ``cp_return_global_position_ids`` keeps positions global under context parallelism."""

    sequence_length: int
    input_pp_rank: int
    output_pp_rank: int
    parallel_context: ParallelContext
    use_doc_masking: bool = True
    cp_return_global_position_ids: bool = True
    cp_zigzag: bool = True

    def __call__(self, examples: List[Dict[str, np.ndarray]]) -> Dict[str, Union[np.ndarray, TensorPointer]]:
        ctx = self.parallel_context
        pp_rank = dist.get_rank(ctx.pp_pg)
        result: Dict[str, Union[np.ndarray, TensorPointer]] = {
            "input_ids": TensorPointer(group_rank=self.input_pp_rank),
            "position_ids": TensorPointer(group_rank=self.input_pp_rank),
            "label_ids": TensorPointer(group_rank=self.output_pp_rank),
            "label_mask": TensorPointer(group_rank=self.output_pp_rank),
        }
        if pp_rank not in (self.input_pp_rank, self.output_pp_rank):
            assert all(len(e) == 0 for e in examples)
            return result
        input_ids = np.vstack([np.asarray(e["input_ids"]) for e in examples])
        batch, length = input_ids.shape
        assert length == self.sequence_length + 1, f"Samples should be of length {self.sequence_length + 1} (seq_len+1), but got {length}"
        if "positions" in examples[0] and self.use_doc_masking:
            positions = np.vstack([np.asarray(e["positions"]) for e in examples])
        else:
            positions = np.broadcast_to(np.arange(length, dtype=np.int64), (batch, length)).copy()
        cp_rank, cp_size = dist.get_rank(ctx.cp_pg), ctx.context_parallel_size
        if pp_rank == self.input_pp_rank:
            result["input_ids"] = _cp_cut(input_ids[:, :-1], cp_rank, cp_size, self.cp_zigzag)
            pos = positions[:, :-1].astype(np.int64)
            result["position_ids"] = _cp_cut(pos, cp_rank, cp_size, self.cp_zigzag)
        if pp_rank == self.output_pp_rank:
            mask = np.ones((batch, self.sequence_length), dtype=np.bool_)
            mask &= positions[:, 1:] != 0
            result["label_ids"] = _cp_cut(input_ids[:, 1:], cp_rank, cp_size, self.cp_zigzag)
            result["label_mask"] = _cp_cut(mask, cp_rank, cp_size, self.cp_zigzag)
        return result


@dataclasses.dataclass
class DataCollatorForSFT:
    """Prompt/completion batches: examples carry ``input_ids``, ``position_ids`` and ``label_mask`` already built by
    ``sft_processing`` (loss only on completion tokens); this collator shifts and distributes them."""

    sequence_length: int
    input_pp_rank: int
    output_pp_rank: int
    parallel_context: ParallelContext

    def __call__(self, examples: List[Dict[str, np.ndarray]]) -> Dict[str, Union[np.ndarray, TensorPointer]]:
        ctx = self.parallel_context
        pp_rank = dist.get_rank(ctx.pp_pg)
        result: Dict[str, Union[np.ndarray, TensorPointer]] = {
            "input_ids": TensorPointer(group_rank=self.input_pp_rank),
            "position_ids": TensorPointer(group_rank=self.input_pp_rank),
            "label_ids": TensorPointer(group_rank=self.output_pp_rank),
            "label_mask": TensorPointer(group_rank=self.output_pp_rank),
        }
        if pp_rank not in (self.input_pp_rank, self.output_pp_rank):
            return result
        input_ids = np.vstack([np.asarray(e["input_ids"]) for e in examples])
        positions = np.vstack([np.asarray(e["position_ids"]) for e in examples])
        label_mask = np.vstack([np.asarray(e["label_mask"]) for e in examples]).astype(np.bool_)
        assert input_ids.shape[1] == self.sequence_length + 1
        if pp_rank == self.input_pp_rank:
            result["input_ids"] = input_ids[:, :-1]
            result["position_ids"] = positions[:, :-1].astype(np.int64)
        if pp_rank == self.output_pp_rank:
            result["label_ids"] = input_ids[:, 1:]
            result["label_mask"] = label_mask[:, 1:] & (positions[:, 1:] != 0)
        return result
