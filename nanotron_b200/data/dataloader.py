"""Synthetic data and dataloader plumbing (parity: reference src/nanotron/data/dataloader.py:25-376).

``dummy_infinite_data_generator`` yields uniform-random token batches shaped like the real collators' output.  The
first pipeline stage receives ``input_ids`` (+ ``input_mask`` or ``position_ids``), the last ``label_ids`` /
``label_mask``; every other entry is a ``TensorPointer``.  With context parallelism each rank keeps its zig-zag slice
of the sequence while ``position_ids`` carry the tokens' global positions.
"""
from __future__ import annotations

from typing import Dict, Generator, Iterator, List, Optional, Union

import numpy as np
import torch
from torch.utils.data import DataLoader

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.config import Config
from nanotron_b200.logging import log_rank
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.context_parallel.zigzag import zigzag_positions, zigzag_slice
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer

logger = logging.get_logger(__name__)


def sanity_check_dataloader(dataloader: Iterator[Dict[str, Union[torch.Tensor, TensorPointer]]], parallel_context: ParallelContext, config: Config) -> Iterator[Dict[str, Union[torch.Tensor, TensorPointer]]]:
    """Move host batches to the device (pinned, non-blocking) and, unless sanity checks are off, verify that inputs
    are identical inside a tensor-parallel group and differ across data-parallel replicas."""
    device = parallel_context.device
    for batch in dataloader:
        out = {}
        for k, v in batch.items():
            if isinstance(v, TensorPointer):
                out[k] = v
                continue
            if isinstance(v, np.ndarray):
                v = torch.from_numpy(v)
            if device.type == "cuda" and v.device.type == "cpu":
                v = v.pin_memory().to(device, non_blocking=True)
            out[k] = v
        if not config.general.ignore_sanity_checks:
            from nanotron_b200.sanity_checks import assert_fail_except_rank_with, assert_tensor_synced_across_pg

            for key, value in sorted(out.items(), key=lambda x: x[0]):
                if isinstance(value, TensorPointer):
                    continue
                if "mask" in key:
                    assert value.dtype == torch.bool or value.dtype.is_floating_point or True
                # same batch on all tp ranks
                assert_tensor_synced_across_pg(tensor=value, pg=parallel_context.tp_pg, msg=lambda err, key=key: f"{key} are not synchronized throughout TP {err}")
        yield out


def dummy_infinite_data_generator(
    micro_batch_size: int,
    sequence_length: int,
    input_pp_rank: int,
    output_pp_rank: int,
    vocab_size: int,
    seed: int,
    parallel_context: ParallelContext,
    use_position_ids: bool = False,
    cp_zigzag: bool = True,
    host_pinned: bool = False,
    skip_batches: int = 0,
):
    """Returns a generator factory.  ``host_pinned=True`` builds every batch in pinned host memory and copies it to
    the device asynchronously (the end-to-end input path); otherwise tokens are drawn directly on the device.
    ``skip_batches``: micro-batches this rank already consumed (a resumed run): they are drawn and dropped, so that the run
    continues with the batch the interrupted one would have seen next (the reference restarts the stream)."""

    def data_generator() -> Generator[Dict[str, Union[torch.Tensor, TensorPointer]], None, None]:
        device = parallel_context.device
        dp_rank = dist.get_rank(parallel_context.dp_pg)
        pp_rank = dist.get_rank(parallel_context.pp_pg)
        cp_rank = dist.get_rank(parallel_context.cp_pg)
        cp_size = parallel_context.cp_pg.size()
        gen_device = "cpu" if host_pinned or device.type == "cpu" else device
        generator = torch.Generator(device=gen_device)
        # same data on every tp / cp rank of a replica, different across dp replicas
        generator.manual_seed(seed * (1 + dp_rank) * (1 + pp_rank * 0))
        if cp_size > 1:
            local_positions = zigzag_positions(sequence_length, cp_rank, cp_size) if cp_zigzag else torch.arange(cp_rank * sequence_length // cp_size, (cp_rank + 1) * sequence_length // cp_size)
        else:
            local_positions = torch.arange(sequence_length)

        def to_device(t):
            if host_pinned and device.type == "cuda":
                return t.pin_memory().to(device, non_blocking=True)
            return t.to(device) if t.device != device else t

        for _ in range(skip_batches):
            torch.randint(0, vocab_size, (micro_batch_size, sequence_length + 1), dtype=torch.long, device=gen_device, generator=generator)
        while True:
            tokens = torch.randint(0, vocab_size, (micro_batch_size, sequence_length + 1), dtype=torch.long, device=gen_device, generator=generator)
            input_ids, label_ids = tokens[:, :-1], tokens[:, 1:]
            if cp_size > 1:
                if cp_zigzag:
                    input_ids = zigzag_slice(input_ids, cp_rank, cp_size, dim=1)
                    label_ids = zigzag_slice(label_ids, cp_rank, cp_size, dim=1)
                else:
                    n = sequence_length // cp_size
                    input_ids = input_ids[:, cp_rank * n : (cp_rank + 1) * n]
                    label_ids = label_ids[:, cp_rank * n : (cp_rank + 1) * n]
            local_len = input_ids.shape[1]
            batch: Dict[str, Union[torch.Tensor, TensorPointer]] = {}
            if pp_rank == input_pp_rank:
                batch["input_ids"] = to_device(input_ids.contiguous())
                if use_position_ids:
                    batch["position_ids"] = to_device(local_positions.unsqueeze(0).expand(micro_batch_size, -1).contiguous())
                else:
                    batch["input_mask"] = torch.ones(micro_batch_size, local_len, dtype=torch.bool, device=device)
            else:
                batch["input_ids"] = TensorPointer(group_rank=input_pp_rank)
                batch["position_ids" if use_position_ids else "input_mask"] = TensorPointer(group_rank=input_pp_rank)
            if pp_rank == output_pp_rank:
                batch["label_ids"] = to_device(label_ids.contiguous())
                batch["label_mask"] = torch.ones(micro_batch_size, local_len, dtype=torch.bool, device=device)
            else:
                batch["label_ids"] = TensorPointer(group_rank=output_pp_rank)
                batch["label_mask"] = TensorPointer(group_rank=output_pp_rank)
            yield batch

    return data_generator


def get_dataloader_worker_init(dp_rank: int):
    """Distinct numpy / python seeds per (dp rank, worker)."""

    def dataloader_worker_init(worker_id):
        import random

        seed = 2**32 - 1 - (dp_rank * 1000 + worker_id)
        np.random.seed(seed % (2**32))
        random.seed(seed)

    return dataloader_worker_init


def get_train_dataloader(
    train_dataset,
    sequence_length: int,
    parallel_context: ParallelContext,
    input_pp_rank: int,
    output_pp_rank: int,
    micro_batch_size: int,
    consumed_train_samples: int,
    dataloader_num_workers: int,
    seed_worker: int,
    dataloader_drop_last: bool = True,
    dataloader_pin_memory: bool = True,
    use_loop_to_round_batch_size: bool = False,
    use_position_ids: bool = False,
    use_doc_masking: bool = True,
    sampler_shuffle: bool = False,
) -> DataLoader:
    """Standard map-style dataloader: dp-sharded sampler (resumable), CLM collator, pinned memory.
    Pipeline ranks that need no data iterate an empty dataset of the same length."""
    from nanotron_b200.data.clm_collator import DataCollatorForCLM, DataCollatorForCLMWithPositionIds
    from nanotron_b200.data.samplers import EmptyInfiniteDataset, get_sampler

    if not isinstance(train_dataset, torch.utils.data.Dataset) and not hasattr(train_dataset, "__getitem__"):
        raise ValueError(f"training requires a map-style dataset, got {type(train_dataset)}")
    pp_rank = dist.get_rank(parallel_context.pp_pg)
    if pp_rank not in (input_pp_rank, output_pp_rank):
        train_dataset = EmptyInfiniteDataset(length=len(train_dataset))
        dataloader_num_workers = 0
    elif hasattr(train_dataset, "with_format"):
        train_dataset = train_dataset.with_format(type="numpy", columns=["input_ids"] + (["positions"] if "positions" in getattr(train_dataset, "column_names", []) else []), output_all_columns=False)
    if use_position_ids:
        collator = DataCollatorForCLMWithPositionIds(sequence_length=sequence_length, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank, parallel_context=parallel_context, use_doc_masking=use_doc_masking)
    else:
        collator = DataCollatorForCLM(sequence_length=sequence_length, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank, parallel_context=parallel_context)
    dp_size = parallel_context.dp_pg.size()
    dp_rank = dist.get_rank(parallel_context.dp_pg)
    sampler = get_sampler(dl_rank=dp_rank, dl_ranks_size=dp_size, train_dataset=train_dataset, seed=seed_worker, use_loop_to_round_batch_size=use_loop_to_round_batch_size, micro_batch_size=micro_batch_size, drop_last=dataloader_drop_last, consumed_train_samples=consumed_train_samples, shuffle=sampler_shuffle)
    return DataLoader(
        train_dataset, batch_size=micro_batch_size, sampler=sampler, collate_fn=collator, drop_last=dataloader_drop_last,
        num_workers=dataloader_num_workers, pin_memory=dataloader_pin_memory and torch.cuda.is_available(),
        worker_init_fn=get_dataloader_worker_init(dp_rank=dp_rank),
    )
