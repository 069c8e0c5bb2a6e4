"""Token samplers over vocabulary-sharded logits (parity: reference src/nanotron/generation/sampler.py).

Each sampler receives ``sharded_logits`` [batch, vocab/tp] on every tensor-parallel rank and returns the same
[batch, 1] token ids on all of them.  Greedy and top-k only exchange their per-shard candidates (2 resp. 2k numbers per
row); top-p and basic sampling gather the full row.  Random draws are made on tp rank 0 and broadcast so ranks agree.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.config.utils_config import SamplerType  # noqa: F401  (re-export)


def _gather_last_dim(x: torch.Tensor, pg) -> torch.Tensor:
    if pg is None or pg.size() == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(pg.size())]
    dist.all_gather(parts, x.contiguous(), group=pg)
    return torch.cat(parts, dim=-1)


def _agree(tokens: torch.Tensor, pg) -> torch.Tensor:
    if pg is not None and pg.size() > 1:
        dist.broadcast(tokens, src=dist.get_global_rank(pg, 0), group=pg)
    return tokens


class Sampler:
    def __call__(self, sharded_logits: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class GreedySampler(Sampler):
    pg: Optional[dist.ProcessGroup]

    def __call__(self, sharded_logits: torch.Tensor) -> torch.Tensor:
        vshard = sharded_logits.shape[-1]
        rank = dist.get_rank(self.pg) if self.pg is not None and self.pg.size() > 1 else 0
        vals, idx = sharded_logits.float().max(dim=-1, keepdim=True)
        idx = idx + rank * vshard
        all_vals = _gather_last_dim(vals, self.pg)  # [b, tp]
        all_idx = _gather_last_dim(idx, self.pg)
        best = all_vals.argmax(dim=-1, keepdim=True)  # first maximum: lowest shard wins ties
        return all_idx.gather(1, best)


@dataclass
class TopKSampler(Sampler):
    pg: Optional[dist.ProcessGroup]
    k: int = 50
    temperature: float = 1.0

    def __call__(self, sharded_logits: torch.Tensor) -> torch.Tensor:
        vshard = sharded_logits.shape[-1]
        rank = dist.get_rank(self.pg) if self.pg is not None and self.pg.size() > 1 else 0
        k_local = min(self.k, vshard)
        vals, idx = torch.topk(sharded_logits.float(), k_local, dim=-1)
        idx = idx + rank * vshard
        all_vals, all_idx = _gather_last_dim(vals, self.pg), _gather_last_dim(idx, self.pg)
        top_vals, pos = torch.topk(all_vals, min(self.k, all_vals.shape[-1]), dim=-1)
        top_idx = all_idx.gather(1, pos)
        probs = torch.softmax(top_vals / self.temperature, dim=-1)
        choice = torch.multinomial(probs, num_samples=1)
        return _agree(top_idx.gather(1, choice), self.pg)


@dataclass
class TopPSampler(Sampler):
    pg: Optional[dist.ProcessGroup]
    p: float = 0.9
    temperature: float = 1.0
    filter_value: float = 0.0
    min_tokens_to_keep: int = 1

    def __call__(self, sharded_logits: torch.Tensor) -> torch.Tensor:
        logits = _gather_last_dim(sharded_logits, self.pg).float()
        probs = torch.softmax(logits / self.temperature, dim=-1)
        sorted_probs, sorted_idx = torch.sort(probs, descending=False, dim=-1)
        cumulative = torch.cumsum(sorted_probs, dim=-1, dtype=torch.float)
        remove_sorted = cumulative <= (1 - self.p)
        if self.min_tokens_to_keep > 1:
            remove_sorted[..., -self.min_tokens_to_keep :] = False
        remove = remove_sorted.scatter(dim=1, index=sorted_idx, src=remove_sorted)
        filtered = probs.masked_fill(remove, self.filter_value)
        return _agree(torch.multinomial(filtered, num_samples=1), self.pg)


@dataclass
class BasicSampler(Sampler):
    """Plain multinomial sampling from the full softmax."""

    pg: Optional[dist.ProcessGroup]

    def __call__(self, sharded_logits: torch.Tensor) -> torch.Tensor:
        logits = _gather_last_dim(sharded_logits, self.pg).float()
        return _agree(torch.multinomial(torch.softmax(logits, dim=-1), num_samples=1), self.pg)
