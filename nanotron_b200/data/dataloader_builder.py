"""Dataloader over a ``Nanoset`` (capability parity: reference src/nanotron/data/dataloader_builder.py:20-82): dp-sharded,
resumable sampler without shuffling (the Nanoset index is already shuffled), causal-LM collator with or without position ids."""
from __future__ import annotations

from torch.utils.data import DataLoader

from nanotron_b200.data.dataloader import get_train_dataloader


def build_nanoset_dataloader(dataset, sequence_length: int, parallel_context, input_pp_rank: int, output_pp_rank: int, micro_batch_size: int,
                             dataloader_num_workers: int, consumed_train_samples: int = 0, dataloader_drop_last: bool = True, dataloader_pin_memory: bool = True,
                             use_position_ids: bool = True, use_doc_masking: bool = True) -> DataLoader:
    return get_train_dataloader(
        train_dataset=dataset, sequence_length=sequence_length, parallel_context=parallel_context, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank,
        micro_batch_size=micro_batch_size, consumed_train_samples=consumed_train_samples, dataloader_num_workers=dataloader_num_workers, seed_worker=0,
        dataloader_drop_last=dataloader_drop_last, dataloader_pin_memory=dataloader_pin_memory, use_position_ids=use_position_ids, use_doc_masking=use_doc_masking,
        sampler_shuffle=False,
    )
