"""Samplers that shard a dataset over data-parallel ranks and can resume mid-epoch
(parity: reference src/nanotron/data/samplers.py)."""
from __future__ import annotations

from typing import Iterator, Optional

import numpy as np
import torch
from torch.utils.data import BatchSampler, Dataset, DistributedSampler, Sampler


class SkipBatchSampler(BatchSampler):
    """Wraps a batch sampler and drops its first ``skip_batches`` batches (resume after ``consumed`` samples)."""

    def __init__(self, batch_sampler: BatchSampler, skip_batches: int, dp_size: int):
        self.batch_sampler = batch_sampler
        self.skip_batches = skip_batches // dp_size if dp_size > 0 else skip_batches
        self.dp_size = dp_size

    @property
    def total_length(self):
        return len(self.batch_sampler)

    def __len__(self):
        return max(0, len(self.batch_sampler) - self.skip_batches)

    def __iter__(self):
        for index, samples in enumerate(self.batch_sampler):
            if index >= self.skip_batches:
                yield samples

    def set_epoch(self, epoch):
        if hasattr(self.batch_sampler, "sampler") and hasattr(self.batch_sampler.sampler, "set_epoch"):
            self.batch_sampler.sampler.set_epoch(epoch)


class DistributedSamplerWithLoop(DistributedSampler):
    """DistributedSampler that loops back to the start so every rank gets full batches."""

    def __init__(self, dataset, batch_size, **kwargs):
        super().__init__(dataset, **kwargs)
        self.batch_size = batch_size

    def __iter__(self):
        indices = list(super().__iter__())
        remainder = 0 if len(indices) % self.batch_size == 0 else self.batch_size - len(indices) % self.batch_size
        start_remainder = 1 if self.rank < len(self.dataset) % self.num_replicas else 0
        indices += indices[start_remainder : start_remainder + remainder]
        return iter(indices)


class EmptyInfiniteDataset:
    """Yields empty examples: given to pipeline ranks that need no data so their dataloader has the right length."""

    def __init__(self, length: int):
        self._length = length

    def __getitem__(self, idx):
        if isinstance(idx, (list, tuple)):
            return [{} for _ in idx]
        return {}

    def __len__(self):
        return self._length


def get_sampler(dl_ranks_size: int, dl_rank: int, train_dataset, consumed_train_samples: int, seed: int = 42, use_loop_to_round_batch_size: bool = False, micro_batch_size: Optional[int] = None, drop_last: bool = True, shuffle: bool = False) -> Optional[Sampler]:
    """Per-dp-rank sampler; ``consumed_train_samples`` (global count) are skipped for resuming."""
    if use_loop_to_round_batch_size:
        assert micro_batch_size is not None
        sampler = DistributedSamplerWithLoop(train_dataset, batch_size=micro_batch_size, num_replicas=dl_ranks_size, rank=dl_rank, seed=seed, drop_last=drop_last)
    else:
        sampler = DistributedSampler(train_dataset, num_replicas=dl_ranks_size, rank=dl_rank, seed=seed, drop_last=drop_last, shuffle=shuffle)
    if consumed_train_samples > 0:
        sampler = SkipBatchSampler(BatchSampler(sampler, batch_size=1, drop_last=False), skip_batches=consumed_train_samples, dp_size=dl_ranks_size)
        return _Flatten(sampler)
    return sampler


class _Flatten(Sampler):
    def __init__(self, batch_sampler):
        self.batch_sampler = batch_sampler

    def __iter__(self):
        for b in self.batch_sampler:
            yield from b

    def __len__(self):
        return len(self.batch_sampler)

    def set_epoch(self, epoch):
        self.batch_sampler.set_epoch(epoch)


# --------------------------------------------------------------------------- Megatron-style samplers
class MegatronPretrainingSampler:
    """Sequential batches of global indices; rank r takes slice r of every global micro-batch."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int, data_parallel_size: int, drop_last: bool = True, global_batch_size: Optional[int] = None, pad_samples_to_global_batch_size: bool = False):
        assert total_samples > 0, f"no sample to consume: {total_samples}"
        assert micro_batch_size > 0 and data_parallel_size > 0
        assert data_parallel_rank < data_parallel_size
        self.total_samples = total_samples
        self.consumed_samples = consumed_samples
        self.micro_batch_size = micro_batch_size
        self.data_parallel_rank = data_parallel_rank
        self.data_parallel_size = data_parallel_size
        self.micro_batch_times_data_parallel_size = micro_batch_size * data_parallel_size
        self.drop_last = drop_last
        self.global_batch_size = global_batch_size
        self.pad_samples_to_global_batch_size = pad_samples_to_global_batch_size

    def __len__(self):
        n = self.total_samples - self.consumed_samples
        if self.drop_last:
            return n // self.micro_batch_times_data_parallel_size
        return (n + self.micro_batch_times_data_parallel_size - 1) // self.micro_batch_times_data_parallel_size

    def get_start_end_idx(self):
        start = self.data_parallel_rank * self.micro_batch_size
        return start, start + self.micro_batch_size

    def __iter__(self):
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.micro_batch_times_data_parallel_size:
                s, e = self.get_start_end_idx()
                yield batch[s:e]
                batch = []
        if len(batch) > 0 and not self.drop_last:
            s, e = self.get_start_end_idx()
            part = batch[s:e]
            if self.pad_samples_to_global_batch_size:
                part = part + [-1] * (self.micro_batch_size - len(part))
            yield part


class MegatronPretrainingRandomSampler(MegatronPretrainingSampler):
    """Each epoch is a seeded permutation of this rank's bucket; resumable through ``consumed_samples``."""

    def __init__(self, *args, seed: int = 0, **kwargs):
        super().__init__(*args, **kwargs)
        self.seed = seed
        self.last_batch_size = self.total_samples % self.micro_batch_times_data_parallel_size

    def __iter__(self):
        active_total = self.total_samples - self.last_batch_size
        epoch = self.consumed_samples // active_total
        current = self.consumed_samples % active_total
        assert current % self.micro_batch_times_data_parallel_size == 0
        bucket_size = (self.total_samples // self.micro_batch_times_data_parallel_size) * self.micro_batch_size
        bucket_offset = current // self.data_parallel_size
        start = self.data_parallel_rank * bucket_size
        g = torch.Generator()
        g.manual_seed(self.seed + epoch)
        perm = torch.randperm(bucket_size, generator=g).tolist()
        idx_range = [start + x for x in perm[bucket_offset:]]
        batch = []
        for idx in idx_range:
            batch.append(idx)
            if len(batch) == self.micro_batch_size:
                self.consumed_samples += self.micro_batch_times_data_parallel_size
                yield batch
                batch = []


class MegatronPretrainingCyclicSampler(MegatronPretrainingSampler):
    """Sequential sampler that wraps around at the end of the dataset (never stops)."""

    def __iter__(self):
        idx = self.consumed_samples
        while True:
            batch = [(idx + i) % self.total_samples for i in range(self.micro_batch_times_data_parallel_size)]
            idx += self.micro_batch_times_data_parallel_size
            s, e = self.get_start_end_idx()
            yield batch[s:e]
