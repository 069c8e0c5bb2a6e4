"""Optimizer / LR-scheduler checkpoints (format parity: reference src/nanotron/serialize/optimizer.py:27-370).

``optimizer/optimizer_config.json`` records the optimizer type, the topology it was saved under and, for ZeRO-1, the
per-parameter dp-rank offsets and original shapes.  State dicts are ``torch.save``d per (pp, [dp,] tp, exp) rank.
Loading supports the same topology (fast path), a different dp size under ZeRO-1 (merge dp shards, re-slice) and a
different tp size (merge + re-shard each state tensor through the parameters' slice maps).
"""
from __future__ import annotations

import json
import warnings
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200 import optim
from nanotron_b200.logging import get_logger, log_rank
from nanotron_b200.optim.zero import ZeroDistributedOptimizer, extract_parallel_ranks_from_shard_path, merge_dp_shard_in_zero1_optimizer
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.serialize.metadata import TensorMetadata
from nanotron_b200.serialize.utils import ObjectType, merge_and_shard_tp_tensors

logger = get_logger(__name__)


def _ep(parallel_context):
    size = parallel_context.expert_parallel_size
    return (dist.get_rank(parallel_context.ep_pg) if size > 1 else 0), size


def optimizer_filename(parallel_context: ParallelContext, is_zero: bool) -> str:
    ep_rank, ep_size = _ep(parallel_context)
    pp, tp, dp = parallel_context.pp_pg, parallel_context.tp_pg, parallel_context.dp_pg
    if is_zero:
        return f"{ObjectType.OPTIMIZER.value}_pp-{dist.get_rank(pp)}-of-{pp.size()}_dp-{dist.get_rank(dp)}-of-{dp.size()}_tp-{dist.get_rank(tp)}-of-{tp.size()}_exp-{ep_rank}-of-{ep_size}.pt"
    return f"{ObjectType.OPTIMIZER.value}_pp-{dist.get_rank(pp)}-of-{pp.size()}_tp-{dist.get_rank(tp)}-of-{tp.size()}_exp-{ep_rank}-of-{ep_size}.pt"


def lr_scheduler_filename(parallel_context: ParallelContext, is_zero: bool) -> str:
    return optimizer_filename(parallel_context, is_zero).replace(ObjectType.OPTIMIZER.value + "_", ObjectType.LR_SCHEDULER.value + "_", 1)


def _is_first_replica(parallel_context: ParallelContext) -> bool:
    """One writer per distinct optimizer state: replicas over context parallelism and over the data-parallel ranks that hold the
    SAME experts are identical, but with expert parallelism laid over the dp axis the dp ranks of different expert ranks are not."""
    if dist.get_rank(parallel_context.cp_pg) > 0:
        return False
    replicas = parallel_context.expert_dp_pg if parallel_context.expert_parallel_size > 1 else parallel_context.dp_pg
    return dist.get_rank(replicas) == 0


def save_optimizer(optimizer: optim.BaseOptimizer, parallel_context: ParallelContext, root_folder: Path):
    if not optimizer.inherit_from(ZeroDistributedOptimizer) and not _is_first_replica(parallel_context):
        return  # identical on every replica: only the first writes
    if optimizer.inherit_from(ZeroDistributedOptimizer) and dist.get_rank(parallel_context.cp_pg) > 0:
        return
    root_folder = Path(root_folder) / "optimizer"
    root_folder.mkdir(exist_ok=True, parents=True)
    if dist.get_rank(parallel_context.world_pg) == 0:
        cfg = {
            "type": str(optimizer.__class__.__name__),
            "parallelism": {
                "tp_size": str(parallel_context.tp_pg.size()),
                "dp_size": str(parallel_context.dp_pg.size()),
                "pp_size": str(parallel_context.pp_pg.size()),
                "expert_parallel_size": str(parallel_context.expert_parallel_size),
            },
            "configs": {},
        }
        if isinstance(optimizer, ZeroDistributedOptimizer):
            cfg["configs"]["param_name_to_dp_rank_offsets"] = {n: {str(r): list(v) for r, v in per.items()} for n, per in optimizer.param_name_to_dp_rank_offsets.items()}
            cfg["configs"]["orig_param_shapes"] = {n: list(p.shape) for g in optimizer.zero_named_param_groups for n, p in g["named_params"]}
        with open(root_folder / "optimizer_config.json", "w") as fo:
            json.dump(cfg, fo)
    torch.save(optimizer.state_dict(), root_folder / optimizer_filename(parallel_context, is_zero=optimizer.inherit_from(ZeroDistributedOptimizer)))


def save_lr_scheduler(lr_scheduler, is_zero, parallel_context: ParallelContext, root_folder: Path):
    if not is_zero and not _is_first_replica(parallel_context):
        return
    if is_zero and dist.get_rank(parallel_context.cp_pg) > 0:
        return
    root_folder = Path(root_folder) / "lr_scheduler"
    root_folder.mkdir(exist_ok=True, parents=True)
    torch.save(lr_scheduler.state_dict(), root_folder / lr_scheduler_filename(parallel_context, is_zero))


def _reshard_state_tensor(full_unsharded: torch.Tensor, param: NanotronParameter) -> torch.Tensor:
    """Cut this rank's shard of an unsharded state tensor following the parameter's slice map."""
    if not (isinstance(param, NanotronParameter) and param.is_sharded):
        return full_unsharded
    info = param.get_sharded_info()
    out = torch.empty(tuple(param.shape) if param.dim() > 0 else (), dtype=full_unsharded.dtype)
    for sp in info.local_global_slices_pairs:
        out[sp.local_slices] = full_unsharded[sp.global_slices]
    return out


@torch.no_grad()
def load_optimizer(optimizer: optim.BaseOptimizer, parallel_context: ParallelContext, root_folder: Path, map_location: Optional[str] = None, param_shard_metadata: Optional[Dict[str, Dict[Tuple[str, str], TensorMetadata]]] = None, model: Optional[nn.Module] = None):
    root_folder = Path(root_folder) / "optimizer"
    with open(root_folder / "optimizer_config.json") as fi:
        ckp_cfg = json.load(fi)
    ckp_pp = int(ckp_cfg["parallelism"]["pp_size"])
    ckp_tp = int(ckp_cfg["parallelism"]["tp_size"])
    ckp_dp = int(ckp_cfg["parallelism"]["dp_size"])
    is_zero_ckp = "ZeroDistributedOptimizer" in ckp_cfg["type"]
    is_zero_now = optimizer.inherit_from(ZeroDistributedOptimizer)
    ckp_ep = int(ckp_cfg["parallelism"].get("expert_parallel_size", 1))
    same_topology = (
        ckp_pp == parallel_context.pp_pg.size() and ckp_tp == parallel_context.tp_pg.size() and ckp_ep == parallel_context.expert_parallel_size
        and (not is_zero_ckp or ckp_dp == parallel_context.dp_pg.size()) and is_zero_ckp == is_zero_now
    )
    if same_topology:
        state_dict = torch.load(root_folder / optimizer_filename(parallel_context, is_zero=is_zero_now), map_location=map_location, weights_only=False)
        optimizer.load_state_dict(state_dict, map_location=map_location)
        return
    if ckp_ep > 1 or parallel_context.expert_parallel_size > 1:
        # the merge below keys shards by (pp, tp) only: states of expert-sharded parameters from different expert ranks would overwrite each other
        raise NotImplementedError(
            f"optimizer states saved with expert_parallel_size={ckp_ep} can only be resumed under the same tp / pp / dp / ep topology "
            f"(now tp={parallel_context.tp_pg.size()} pp={parallel_context.pp_pg.size()} dp={parallel_context.dp_pg.size()} ep={parallel_context.expert_parallel_size}); "
            "resume with `checkpoints.load_optimizer: false` or under the saved topology"
        )
    assert model is not None, "loading optimizer states under a different topology needs the model (for the parameters' slice maps)"
    # 1) unshard over dp (ZeRO) -> {(pp, tp): state dict with full-shard tensors}
    if is_zero_ckp:
        shard_paths = sorted(root_folder.glob(f"{ObjectType.OPTIMIZER.value}_pp-*-of-{ckp_pp}_dp-*-of-{ckp_dp}_tp-*-of-{ckp_tp}_exp-*.pt"))
        per_pp_tp = merge_dp_shard_in_zero1_optimizer(model, ckp_cfg, shard_paths, parallel_context, map_location="cpu")
    else:
        per_pp_tp = {}
        for p in sorted(root_folder.glob(f"{ObjectType.OPTIMIZER.value}_pp-*-of-{ckp_pp}_tp-*-of-{ckp_tp}_exp-*.pt")):
            per_pp_tp[extract_parallel_ranks_from_shard_path(p, is_zero1=False)] = torch.load(p, map_location="cpu", weights_only=False)
    # 2) gather each named state across the checkpoint's tp ranks into unsharded tensors
    name_to_param = dict(model.get_named_params_with_correct_tied()) if hasattr(model, "get_named_params_with_correct_tied") else dict(model.named_parameters())
    new_sd = optimizer.state_dict()
    new_names = new_sd["names"]
    state_keys = ["exp_avg", "exp_avg_sq"]
    new_state = {}
    my_dp = dist.get_rank(parallel_context.dp_pg)
    my_tp = dist.get_rank(parallel_context.tp_pg)
    my_pp = dist.get_rank(parallel_context.pp_pg)
    same_tp = ckp_tp == parallel_context.tp_pg.size()

    def holders(name):
        """Checkpoint state dicts that hold ``name``, as [((pp, tp), state dict, index)].  With an unchanged tp size only this
        rank's own tp shard qualifies (every tp rank of the checkpoint holds the name, each with different data); the
        stage that matches this rank's pipeline rank comes first (a tied parameter lives on two stages)."""
        found = []
        for (pp_rank, tp_rank), sd in per_pp_tp.items():
            if same_tp and tp_rank != my_tp:
                continue
            ckp_idx = next((k for k, v in sd["names"].items() if v == name), None)
            if ckp_idx is not None:
                found.append(((pp_rank, tp_rank), sd, ckp_idx))
        found.sort(key=lambda e: (e[0][0] != my_pp, e[0]))
        return found

    # the tensors the inner optimizer really steps (ZeRO: this rank's slice of each master, in whatever shape the optimizer holds it):
    # torch numbers them consecutively over the parameter groups, which is the numbering of ``names``
    stepped = [p for group in optimizer.get_base_optimizer().param_groups for p in group["params"]]

    def shaped_like_stepped(idx, t: torch.Tensor) -> torch.Tensor:
        target = stepped[idx] if isinstance(idx, int) and idx < len(stepped) else None
        return t.view(target.shape) if target is not None and target.numel() == t.numel() else t

    for idx, name in new_names.items():
        param = name_to_param[name]
        found = holders(name)
        assert found, f"optimizer state of {name} not found in checkpoint"
        shards = [(key[1], sd["state"][ckp_idx]) for key, sd, ckp_idx in found]
        step = shards[0][1]["step"]
        entry = {"step": step}
        for sk in state_keys:
            if isinstance(param, NanotronParameter) and param.is_sharded and ckp_tp != parallel_context.tp_pg.size():
                assert param_shard_metadata is not None and name in param_shard_metadata or True
                info = param.get_sharded_info()
                unsharded = torch.zeros(tuple(info.unsharded_shape), dtype=torch.float32)
                # slice maps of the checkpoint shards were collected while loading the weights
                metas = (param_shard_metadata or {}).get(name, {})
                for tp_rank, st in shards:
                    meta = next((m for (pp_s, tp_s), m in metas.items() if int(tp_s) == int(tp_rank)), None)
                    assert meta is not None, f"missing slice map of {name} tp shard {tp_rank}; load the weights first with param_shard_metadata"
                    shard_t = st[sk].float()
                    for sp in meta.local_global_slices_pairs:
                        unsharded[sp.global_slices] = shard_t.view(_local_shape(meta))[sp.local_slices]
                local = _reshard_state_tensor(unsharded, param)
            else:
                local = shards[0][1][sk].float().view(param.shape)
            if is_zero_now:
                rng = optimizer.param_name_to_dp_rank_offsets[name].get(my_dp)
                local = local.reshape(-1)[rng[0] : rng[1]] if rng is not None else local.reshape(-1)[0:0]
            entry[sk] = shaped_like_stepped(idx, local.clone())
        new_state[idx] = entry
    new_sd["state"] = new_state
    if "gradient_accumulator" in new_sd:
        ga = {}
        for name in new_sd["gradient_accumulator"]:
            param = name_to_param[name]
            src = None
            for (pp_rank, tp_rank), sd in sorted(per_pp_tp.items(), key=lambda e: (e[0][0] != my_pp, e[0])):
                if same_tp and tp_rank != my_tp:
                    continue
                if "gradient_accumulator" in sd and name in sd["gradient_accumulator"]:
                    src = sd["gradient_accumulator"][name]
                    break
            if src is None or not same_tp:
                # masters can always be rebuilt from the (already loaded) parameters
                full = param.detach().float().cpu()
            else:
                full = src.float().view(param.shape)
            if is_zero_now:
                rng = optimizer.param_name_to_dp_rank_offsets[name].get(my_dp)
                full = full.reshape(-1)[rng[0] : rng[1]] if rng is not None else full.reshape(-1)[0:0]
            ga[name] = full
        new_sd["gradient_accumulator"] = ga
    optimizer.load_state_dict(new_sd, map_location=map_location)


def _local_shape(meta: TensorMetadata):
    """Shape of the shard described by a slice map: per dimension the largest explicit local stop, or, when the local slice
    is the whole dimension (``slice(None)``), the extent of the matching global slice."""
    shape = []
    pairs = meta.local_global_slices_pairs
    ndim = len(meta.unsharded_shape)
    for d in range(ndim):
        extent = 0
        for sp in pairs:
            ls, gs = sp.local_slices[d], sp.global_slices[d]
            if ls.stop is not None:
                extent = max(extent, ls.stop)
            else:
                g0 = gs.start or 0
                g1 = gs.stop if gs.stop is not None else meta.unsharded_shape[d]
                extent = max(extent, (ls.start or 0) + (g1 - g0))
        shape.append(extent)
    return tuple(shape)


def load_lr_scheduler(lr_scheduler, is_zero, parallel_context: ParallelContext, root_folder: Path):
    root_folder = Path(root_folder) / "lr_scheduler"
    path = root_folder / lr_scheduler_filename(parallel_context, is_zero)
    if not path.exists():
        candidates = sorted(root_folder.glob(f"{ObjectType.LR_SCHEDULER.value}_*.pt"))
        assert candidates, f"no lr scheduler state in {root_folder}"
        path = candidates[0]
    state_dict = torch.load(path, weights_only=False)
    lr_scheduler.load_state_dict(state_dict)
    # Put the learning rates the scheduler had computed for the next step back into the optimizer.  (The reference calls
    # ``_initial_step()`` here, serialize/optimizer.py:369-370, which advances the schedule by one extra step on every resume.)
    for group, lr in zip(lr_scheduler.optimizer.param_groups, lr_scheduler.get_last_lr()):
        group["lr"] = lr
