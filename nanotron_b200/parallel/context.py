"""Process-group topology.

Same attribute names and rank-grid order as the reference (reference
src/nanotron/parallel/context.py:12-183): the grid is ordered slowest to fastest
``["ep", "pp", "dp", "cp", "tp"]`` so tensor-parallel peers are adjacent GPUs on the
NVSwitch fabric.  Two deliberate differences:

* backend is ``nccl`` or ``gloo`` (CPU), chosen automatically when not given;
* expert parallelism is an *overlay on the data-parallel axis*: ``world = pp*dp*cp*tp``
  and ``ep`` must divide ``dp``.  Consecutive dp ranks form one expert-parallel group,
  ranks with the same ep rank form ``expert_dp_pg`` (the group expert gradients are
  averaged over).  The leading "ep" axis of ``world_rank_matrix`` therefore has length 1
  and ``get_global_rank(ep_rank, ...)`` ignores its first argument.  With this, EP=8 x DP=8
  runs on 8 GPUs, which a separate ep axis cannot express.
"""
from __future__ import annotations

import os
from typing import Dict, Literal, Optional

import numpy as np
import torch

import nanotron_b200.distributed as dist

DistributedBackend = Literal["gloo", "nccl"]


class ParallelContext:
    def __init__(
        self,
        tensor_parallel_size: int,
        pipeline_parallel_size: int,
        data_parallel_size: int,
        context_parallel_size: int = 1,
        expert_parallel_size: int = 1,
        backend: Optional[DistributedBackend] = None,
    ):
        world_size = int(os.environ.get("WORLD_SIZE", "1"))
        local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", str(min(world_size, 8))))
        tp, pp, dp, cp, ep = (
            tensor_parallel_size,
            pipeline_parallel_size,
            data_parallel_size,
            context_parallel_size,
            expert_parallel_size,
        )
        assert tp * pp * cp * dp == world_size, f"TP*CP*DP*PP={tp}*{cp}*{dp}*{pp}={tp*pp*cp*dp} != WORLD_SIZE={world_size}"
        assert dp % ep == 0, f"expert_parallel_size={ep} must divide data_parallel_size={dp}"
        self.tensor_parallel_size = tp
        self.pipeline_parallel_size = pp
        self.data_parallel_size = dp
        self.context_parallel_size = cp
        self.expert_parallel_size = ep
        self.world_size = world_size
        self.local_world_size = local_world_size
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        assert backend in ("nccl", "gloo"), f"unsupported backend {backend}"
        self.backend = backend
        self.set_device()
        if not dist.is_initialized():
            dist.initialize_torch_distributed(backend)
        self.world_pg = dist.new_group(ranks=list(range(world_size)), backend=dist.get_backend())
        self._init_parallel_groups()

    # ------------------------------------------------------------------ groups
    def _init_parallel_groups(self):
        tp, pp, dp, cp, ep = (
            self.tensor_parallel_size,
            self.pipeline_parallel_size,
            self.data_parallel_size,
            self.context_parallel_size,
            self.expert_parallel_size,
        )
        ranks = np.arange(self.world_size).reshape((1, pp, dp, cp, tp))
        self.world_ranks_to_pg: Dict[tuple, dist.ProcessGroup] = {}
        node = min(self.local_world_size, self.world_size)
        if self.world_size % node == 0:
            self.local_pg = self.create_new_group(ranks.reshape((-1, node)))
        else:
            self.local_pg = self.world_pg
        self.tp_pg = self.create_new_group(ranks.reshape((-1, tp)))
        self.cp_pg = self.create_new_group(ranks.transpose((4, 0, 1, 2, 3)).reshape((-1, cp)))
        self.dp_pg = self.create_new_group(ranks.transpose((3, 4, 0, 1, 2)).reshape((-1, dp)))
        pp_groups = ranks.transpose((2, 3, 4, 0, 1)).reshape((-1, pp))
        self.pp_pg = self.create_new_group(pp_groups)
        if pp > 1:
            # pipeline traffic: one process group per direction (activations forward, gradients backward), see pipeline_parallel/p2p.py
            from nanotron_b200.parallel.pipeline_parallel.p2p import register_lanes

            self.pp_lane_pgs = tuple(self._create_private_group(pp_groups) for _ in range(2))
            register_lanes(self.pp_pg, *self.pp_lane_pgs)
        # expert parallel overlay: dp axis split as (dp // ep, ep)
        r6 = ranks.reshape((pp, dp // ep, ep, cp, tp))
        self.ep_pg = self.create_new_group(r6.transpose((0, 1, 3, 4, 2)).reshape((-1, ep)))
        self.expert_dp_pg = self.create_new_group(r6.transpose((0, 2, 3, 4, 1)).reshape((-1, dp // ep)))
        self.mp_pg = self.create_new_group(
            [ranks[:, :, d, c, :].reshape(-1) for c in range(cp) for d in range(dp)]
        )
        self.dp_cp_pg = self.create_new_group(
            [ranks[0, p, :, :, t].reshape(-1) for t in range(tp) for p in range(pp)]
        )
        self.tp_and_ep_pg = self.create_new_group(
            [r6[p, g, :, c, :].reshape(-1) for c in range(cp) for p in range(pp) for g in range(dp // ep)]
        )
        self.world_rank_matrix: np.ndarray = ranks
        self.parallel_order = ["ep", "pp", "dp", "cp", "tp"]

    def create_new_group(self, all_groups_ranks) -> dist.ProcessGroup:
        """Create (or reuse) every listed group on every rank; return the one holding this rank."""
        rank = int(os.environ.get("RANK", "0"))
        mine = None
        for group_ranks in all_groups_ranks:
            key = tuple(sorted(int(r) for r in group_ranks))
            if key not in self.world_ranks_to_pg:
                self.world_ranks_to_pg[key] = dist.new_group(ranks=list(key), backend=dist.get_backend())
            if rank in key:
                mine = self.world_ranks_to_pg[key]
        return mine

    def _create_private_group(self, all_groups_ranks) -> dist.ProcessGroup:
        """Like ``create_new_group`` but never shared with another axis that happens to span the same ranks."""
        rank = int(os.environ.get("RANK", "0"))
        mine = None
        for group_ranks in all_groups_ranks:
            key = sorted(int(r) for r in group_ranks)
            g = dist.new_group(ranks=key, backend=dist.get_backend())
            if rank in key:
                mine = g
        return mine

    # ------------------------------------------------------------------ misc
    def set_device(self):
        if self.backend == "nccl":
            local_rank = int(os.getenv("LOCAL_RANK", "0"))
            torch.cuda.set_device(local_rank % torch.cuda.device_count())

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", torch.cuda.current_device()) if self.backend == "nccl" else torch.device("cpu")

    def get_local_ranks(self, world_rank: int) -> Dict[str, int]:
        idx = np.where(self.world_rank_matrix == world_rank)
        out = {ax: int(idx[i].item()) for i, ax in enumerate(self.parallel_order)}
        out["ep"] = out["dp"] % self.expert_parallel_size
        return out

    def get_global_rank(self, ep_rank: int, pp_rank: int, dp_rank: int, cp_rank: int, tp_rank: int) -> np.int64:
        """World rank at the given coordinates (``ep_rank`` is implied by ``dp_rank`` and ignored)."""
        return self.world_rank_matrix[0, pp_rank, dp_rank, cp_rank, tp_rank]

    def destroy(self):
        if not dist.is_initialized():
            return
        dist.barrier()
        dist.destroy_process_group()
        dist.get_rank.cache_clear()
        dist.get_global_rank.cache_clear()
