"""Per-rank RNG state files ``random/tp-T-of-N_dp-D-of-M_pp-P-of-K.pt`` (parity: reference src/nanotron/serialize/random.py)."""
from pathlib import Path

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.random import RandomStates


def _file(parallel_context: ParallelContext, root_folder: Path) -> Path:
    return (
        Path(root_folder)
        / "random"
        / f"tp-{dist.get_rank(parallel_context.tp_pg)}-of-{parallel_context.tp_pg.size()}_dp-{dist.get_rank(parallel_context.dp_pg)}-of-{parallel_context.dp_pg.size()}_pp-{dist.get_rank(parallel_context.pp_pg)}-of-{parallel_context.pp_pg.size()}.pt"
    )


def save_random_states(random_states: RandomStates, parallel_context: ParallelContext, root_folder: Path):
    """Every rank saves its own states."""
    path = _file(parallel_context, root_folder)
    path.parent.mkdir(exist_ok=True, parents=True)
    torch.save(random_states, path)


def load_random_states(parallel_context: ParallelContext, root_folder: Path) -> RandomStates:
    return torch.load(_file(parallel_context, root_folder), weights_only=False)
