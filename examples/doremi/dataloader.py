"""Domain-weighted data loading for DoReMi
(capability parity: reference examples/doremi/doremi/dataloader.py -- ``CombinedDataset``, ``DistributedSamplerForDoReMi``,
``DataCollatorForCLM``, ``get_dataloader`` -- and examples/doremi/doremi/utils.py ``compute_domain_weights_based_on_token_count``).

Every domain is a dataset of its own.  For each global batch the sampler turns the current domain weights into whole-number
quotas (every domain keeps at least one sample, so its excess loss stays observable), takes the next ``quota[d]`` items of every
domain's order, mixes them with a step-seeded permutation and hands every data-parallel rank its contiguous part, one micro-batch
at a time.  All ranks run the same arithmetic on the same weights, so no communication is needed to agree on the batch.

The sampler is resumable (``state_dict`` / ``load_state_dict``) and keeps going after a domain is exhausted by starting a new
pass over that domain (``on_exhausted="wrap"``), or stops the epoch there (``"stop"``, what the reference does).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterator, List, Optional, Sequence, Union

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

from nanotron_b200 import distributed as dist
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer


def apportion(weights: Sequence[float], total: int, floor: int = 1, rng: Optional[np.random.Generator] = None) -> List[int]:
    """Whole-number quotas that sum to ``total``, proportional to ``weights``, none below ``floor``.

    Starts from the rounded-down shares and then moves single samples to (from) the domain that is furthest below (above) its
    exact share; ties go to a random domain when ``rng`` is given (so that no domain is favoured batch after batch), else to the
    first."""
    w = np.asarray(weights, dtype=np.float64)
    n = w.size
    if total < n * floor:
        raise ValueError(f"{total} samples cannot give {n} domains {floor} each")
    if (w < 0).any() or w.sum() <= 0:
        raise ValueError("domain weights must be non-negative and not all zero")
    exact = w / w.sum() * total
    counts = np.maximum(np.floor(exact).astype(np.int64), floor)
    order = rng.permutation(n) if rng is not None else np.arange(n)
    while counts.sum() != total:
        gap = (exact - counts)[order]  # > 0: owed samples
        if counts.sum() < total:
            counts[order[int(np.argmax(gap))]] += 1
        else:
            can_give = counts[order] > floor
            gap = np.where(can_give, gap, np.inf)
            counts[order[int(np.argmin(gap))]] -= 1
    return [int(c) for c in counts]


def domain_weights_from_token_count(datasets: Sequence[Dataset], tokens_per_item: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Weights proportional to the size of every domain: the sampling under which all domains run out at the same time."""
    sizes = [len(d) * (tokens_per_item[i] if tokens_per_item is not None else 1) for i, d in enumerate(datasets)]
    t = torch.tensor(sizes, dtype=torch.float64)
    return (t / t.sum()).float()


class CombinedDataset(Dataset):
    """The domains behind one index space: item ``i`` of domain ``d`` has index ``offsets[d] + i`` and comes back with ``d``."""

    def __init__(self, datasets: Sequence[Dataset]):
        self.datasets = list(datasets)
        self.lengths = [len(d) for d in self.datasets]
        self.offsets = np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int64)

    def __len__(self) -> int:
        return int(self.offsets[-1])

    def locate(self, index: int):
        d = int(np.searchsorted(self.offsets, index, side="right") - 1)
        return d, int(index - self.offsets[d])

    def __getitem__(self, index: int) -> Dict[str, Union[np.ndarray, int]]:
        d, i = self.locate(int(index))
        item = self.datasets[d][i]
        ids = item["input_ids"] if isinstance(item, dict) else item
        return {"input_ids": np.asarray(ids), "domain_idx": d}


class DomainWeightedSampler:
    """Batch sampler: yields the indices (into a ``CombinedDataset``) of one micro-batch of this data-parallel rank.

    ``weights_fn`` is read once per global batch; it returns the domain weights (a tensor or a sequence) that this batch follows.
    """

    def __init__(self, lengths: Sequence[int], micro_batch_size: int, num_microbatches: int, dp_size: int, dp_rank: int,
                 weights_fn: Callable[[], Sequence[float]], seed: int = 42, shuffle: bool = True, on_exhausted: str = "wrap"):
        assert on_exhausted in ("wrap", "stop")
        assert 0 <= dp_rank < dp_size
        self.lengths = [int(n) for n in lengths]
        self.offsets = np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int64)
        self.micro_batch_size, self.num_microbatches = micro_batch_size, num_microbatches
        self.dp_size, self.dp_rank = dp_size, dp_rank
        self.weights_fn, self.seed, self.shuffle, self.on_exhausted = weights_fn, seed, shuffle, on_exhausted
        self.global_batch_size = micro_batch_size * num_microbatches * dp_size
        if self.global_batch_size < len(self.lengths):
            raise ValueError(f"a global batch of {self.global_batch_size} cannot hold one sample of each of {len(self.lengths)} domains")
        self.step = 0  # global batches drawn so far
        self.cursors = [0] * len(self.lengths)  # position inside the current pass over every domain
        self.passes = [0] * len(self.lengths)
        self._orders: Dict[int, np.ndarray] = {}
        self.last_quotas: Optional[List[int]] = None

    # the order of a domain in one pass is a function of (seed, domain, pass): nothing but counters has to be saved
    def _order(self, d: int) -> np.ndarray:
        key = d
        if key not in self._orders or self._orders[key][0] != self.passes[d]:
            if self.shuffle:
                perm = np.random.default_rng([self.seed, d, self.passes[d]]).permutation(self.lengths[d])
            else:
                perm = np.arange(self.lengths[d])
            self._orders[key] = (self.passes[d], perm)
        return self._orders[key][1]

    def _take(self, d: int, count: int) -> List[int]:
        out: List[int] = []
        while count > 0:
            left = self.lengths[d] - self.cursors[d]
            if left == 0:
                if self.on_exhausted == "stop":
                    raise StopIteration(f"domain {d} ran out of samples")
                self.passes[d] += 1
                self.cursors[d] = 0
                continue
            n = min(left, count)
            order = self._order(d)
            out.extend((order[self.cursors[d] : self.cursors[d] + n] + self.offsets[d]).tolist())
            self.cursors[d] += n
            count -= n
        return out

    def global_batch(self) -> List[int]:
        """Indices of the next global batch (the same list on every rank)."""
        weights = self.weights_fn()
        weights = weights.detach().float().cpu().tolist() if isinstance(weights, torch.Tensor) else list(weights)
        assert len(weights) == len(self.lengths), "one weight per domain"
        rng = np.random.default_rng([self.seed, 7919, self.step])
        quotas = apportion(weights, self.global_batch_size, floor=1, rng=rng)
        self.last_quotas = quotas
        batch: List[int] = []
        for d, q in enumerate(quotas):
            batch.extend(self._take(d, q))
        mixed = rng.permutation(len(batch))  # every rank and every micro-batch sees a mixture of the domains
        self.step += 1
        return [batch[i] for i in mixed]

    def __iter__(self) -> Iterator[List[int]]:
        per_rank = self.micro_batch_size * self.num_microbatches
        while True:
            try:
                batch = self.global_batch()
            except StopIteration:
                return
            mine = batch[self.dp_rank * per_rank : (self.dp_rank + 1) * per_rank]
            for i in range(0, per_rank, self.micro_batch_size):
                yield mine[i : i + self.micro_batch_size]

    def state_dict(self) -> Dict[str, object]:
        return {"step": self.step, "cursors": list(self.cursors), "passes": list(self.passes)}

    def load_state_dict(self, state: Dict[str, object]) -> None:
        self.step, self.cursors, self.passes = int(state["step"]), list(state["cursors"]), list(state["passes"])
        self._orders.clear()


class DoReMiCollator:
    """``sequence_length + 1`` token ids per item -> the micro-batch dict of the Llama models of this example, plus ``domain_idxs``
    [b].  On a pipeline rank that consumes neither inputs nor labels every key is a ``TensorPointer``."""

    def __init__(self, sequence_length: int, input_pp_rank: int, output_pp_rank: int, parallel_context):
        self.sequence_length, self.input_pp_rank, self.output_pp_rank, self.ctx = sequence_length, input_pp_rank, output_pp_rank, parallel_context

    def __call__(self, items: List[Dict[str, Union[np.ndarray, int]]]) -> Dict[str, Union[torch.Tensor, TensorPointer]]:
        pp_rank = dist.get_rank(self.ctx.pp_pg)
        out: Dict[str, Union[torch.Tensor, TensorPointer]] = {}
        ids = torch.as_tensor(np.stack([np.asarray(it["input_ids"]) for it in items]), dtype=torch.long)
        assert ids.shape[1] == self.sequence_length + 1, f"items must hold sequence_length + 1 = {self.sequence_length + 1} tokens, got {ids.shape[1]}"
        b = ids.shape[0]
        if pp_rank == self.input_pp_rank:
            out["input_ids"] = ids[:, :-1].contiguous()
            out["input_mask"] = torch.ones(b, self.sequence_length, dtype=torch.bool)
        else:
            out["input_ids"] = out["input_mask"] = TensorPointer(group_rank=self.input_pp_rank)
        if pp_rank == self.output_pp_rank:
            out["label_ids"] = ids[:, 1:].contiguous()
            out["label_mask"] = torch.ones(b, self.sequence_length, dtype=torch.bool)
            out["domain_idxs"] = torch.as_tensor([int(it["domain_idx"]) for it in items], dtype=torch.long)
        else:
            out["label_ids"] = out["label_mask"] = out["domain_idxs"] = TensorPointer(group_rank=self.output_pp_rank)
        return out


def get_dataloader(trainer, datasets: Sequence[Dataset], weights_fn: Callable[[], Sequence[float]], seed: Optional[int] = None,
                   on_exhausted: str = "wrap", sampler_state: Optional[Dict[str, object]] = None) -> DataLoader:
    """The dataloader of one data stage; ``trainer.doremi_sampler`` keeps the sampler so that its state can be saved."""
    from nanotron_b200.parallel.pipeline_parallel.utils import get_input_output_pp_ranks

    ctx = trainer.parallel_context
    combined = CombinedDataset(datasets)
    sampler = DomainWeightedSampler(
        combined.lengths, micro_batch_size=trainer.micro_batch_size, num_microbatches=trainer.n_micro_batches_per_batch,
        dp_size=ctx.dp_pg.size(), dp_rank=dist.get_rank(ctx.dp_pg), weights_fn=weights_fn,
        seed=trainer.config.data_stages[0].data.seed if seed is None else seed, on_exhausted=on_exhausted,
    )
    if sampler_state is not None:
        sampler.load_state_dict(sampler_state)
    trainer.doremi_sampler = sampler
    input_pp_rank, output_pp_rank = get_input_output_pp_ranks(model=trainer.unwrapped_model)
    collator = DoReMiCollator(trainer.sequence_length, input_pp_rank, output_pp_rank, ctx)
    # one worker-less loader: the sampler has to read the weights of the step that is about to run, not of a prefetched future
    return DataLoader(combined, batch_sampler=sampler, collate_fn=collator, num_workers=0, pin_memory=ctx.device.type == "cuda")
