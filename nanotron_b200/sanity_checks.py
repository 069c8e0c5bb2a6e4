"""Runtime invariants checked around each phase of a training step when ``general.ignore_sanity_checks`` is False
(parity: reference src/nanotron/sanity_checks.py:19-322).  These stand in for a race detector: replicas that drift,
gradients that vanish or explode, and stale buffers are caught at the step where they appear."""
from __future__ import annotations

from contextlib import contextmanager
from typing import Callable, Optional

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging, optim
from nanotron_b200.logging import get_logger, log_rank
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter
from nanotron_b200.parallel.tied_parameters import get_tied_id_to_param

logger = get_logger(__name__)


def assert_tensor_synced_across_pg(tensor: torch.Tensor, pg: dist.ProcessGroup, msg: Optional[Callable[[str], str]] = None, reference_rank: int = 0):
    """Raise if ``tensor`` differs bitwise from ``reference_rank``'s copy."""
    if pg is None or pg.size() == 1:
        return
    if dist.get_rank(pg) == reference_rank:
        ref = tensor.detach().clone()
    else:
        ref = torch.empty_like(tensor)
    dist.broadcast(ref, src=dist.get_global_rank(pg, reference_rank), group=pg)
    try:
        torch.testing.assert_close(tensor.detach(), ref, atol=0, rtol=0)
    except AssertionError as e:
        raise AssertionError(msg(str(e)) if msg else str(e))


@contextmanager
def assert_fail_except_rank_with(exception_class, rank_exception, pg):
    try:
        yield
    except exception_class:
        if rank_exception == dist.get_rank(pg):
            raise AssertionError(f"Expected rank {rank_exception} to not raise {exception_class}.")
    else:
        if rank_exception != dist.get_rank(pg):
            raise AssertionError(f"Expected {exception_class} to be raised on every rank but {rank_exception}")


def _is_expert(param, parallel_context) -> bool:
    return isinstance(param, NanotronParameter) and param.is_sharded and param.get_sharded_info().is_expert_sharded(parallel_context)


def _replica_group(param, parallel_context):
    return parallel_context.expert_dp_pg if _is_expert(param, parallel_context) else parallel_context.dp_cp_pg


def before_tbi_sanity_checks(config, parallel_context: ParallelContext, unwrapped_model, grad_accumulator, lr_scheduler) -> None:
    if config.general.ignore_sanity_checks:
        return
    # parameters equal across data-parallel replicas
    for name, param in sorted(unwrapped_model.named_parameters(), key=lambda x: x[0]):
        assert_tensor_synced_across_pg(param, _replica_group(param, parallel_context), msg=lambda err, name=name: f"{name} are not synchronized across DP {err}")
    # tied parameters equal inside their tie group
    for (name, ranks), param in sorted(get_tied_id_to_param(list(unwrapped_model.parameters()), unwrapped_model).items(), key=lambda x: x[0]):
        group = parallel_context.world_ranks_to_pg[tuple(sorted(ranks))]
        assert_tensor_synced_across_pg(param, group, msg=lambda err, name=name: f"[Before train] Tied weights {name} are not synchronized. {err}")
    # no stale gradients
    for name, param in unwrapped_model.named_parameters():
        if param.grad is not None:
            torch.testing.assert_close(param.grad, torch.zeros_like(param.grad), atol=0, rtol=0, msg=f"Grad of {name} is not zero before the step")
    if grad_accumulator is not None:
        buf = grad_accumulator._contiguous_fp32_grad_buffer
        assert not bool(buf.any()), "fp32 gradient buffer is not zero before the step"
    # optimizer lr == scheduler lr
    if lr_scheduler is not None:
        expected = lr_scheduler.get_last_lr()
        for i, g in enumerate(lr_scheduler.optimizer.param_groups):
            assert abs(float(g["lr"]) - float(expected[i])) < 1e-12, f"param group {i}: optimizer lr {g['lr']} != scheduler lr {expected[i]}"
    unwrapped_model.before_tbi_sanity_checks()


def after_tbi_sanity_checks(config, parallel_context: ParallelContext, unwrapped_model, grad_accumulator) -> None:
    if config.general.ignore_sanity_checks:
        return
    for name, param in unwrapped_model.named_parameters():
        if not param.requires_grad:
            continue
        grad = grad_accumulator.get_grad_buffer(name=_canonical(name, param, unwrapped_model)) if grad_accumulator is not None else param.grad
        if grad is None:
            log_rank(f"Process rank { dist.get_rank(parallel_context.world_pg)}/{parallel_context.world_pg.size()}: {name} is missing gradient", logger=logger, level=logging.ERROR)
            raise AssertionError(f"{name} is missing gradient")
        if not bool(torch.isfinite(grad).all()):
            raise ValueError(f"Gradient of {name} contains NaN or Inf")
    unwrapped_model.after_tbi_sanity_checks()


def _canonical(name, param, model):
    if isinstance(param, NanotronParameter) and param.is_tied:
        return param.get_tied_info().get_full_name_from_module_id_to_prefix(model.module_id_to_prefix)
    return name


def before_optim_step_sanity_checks(config, parallel_context: ParallelContext, unwrapped_model, grad_accumulator, optimizer) -> None:
    if config.general.ignore_sanity_checks:
        return
    zero = optimizer is not None and optimizer.inherit_from(optim.ZeroDistributedOptimizer)
    # After the in-place reduce-scatter of ZeRO-1 a gradient is only meaningful on the slice its rank optimises, and the members of
    # a tie group (two pipeline stages, say) own different slices of the same weight: whole tensors cannot be compared then.
    # Members on the same stage (tensor-parallel replicas) lay their buffers out identically and own the same slices: those stay comparable.
    sliced = zero and parallel_context.dp_pg.size() > 1
    for (name, ranks), param in sorted(get_tied_id_to_param(list(unwrapped_model.parameters()), unwrapped_model).items(), key=lambda x: x[0]):
        if not param.requires_grad:
            continue
        if sliced and len({parallel_context.get_local_ranks(world_rank=r)["pp"] for r in ranks}) > 1:
            continue
        grad = grad_accumulator.get_grad_buffer(name=name) if grad_accumulator is not None else param.grad
        group = parallel_context.world_ranks_to_pg[tuple(sorted(ranks))]
        assert_tensor_synced_across_pg(grad, group, msg=lambda err, name=name: f"[Before optimizer step] Tied weights grads for {name} are not synchronized. {err}")
    if not zero:
        for name, param in sorted(unwrapped_model.named_parameters(), key=lambda x: x[0]):
            if not param.requires_grad:
                continue
            grad = grad_accumulator.get_grad_buffer(name=_canonical(name, param, unwrapped_model)) if grad_accumulator is not None else param.grad
            assert_tensor_synced_across_pg(grad, _replica_group(param, parallel_context), msg=lambda err, name=name: f"[Before optimizer step] weights grads for {name} are not synchronized across DP. {err}")
    for name, param in sorted(unwrapped_model.named_parameters(), key=lambda x: x[0]):
        assert_tensor_synced_across_pg(param, _replica_group(param, parallel_context), msg=lambda err, name=name: f"{name} are not synchronized across DP {err}")
    if optimizer is not None and not zero:
        # replicas of an optimizer state are the replicas of its parameter: all of dp, except for experts (their dp ranks of other
        # expert ranks hold other experts)
        by_name = dict(unwrapped_model.get_named_params_with_correct_tied()) if hasattr(unwrapped_model, "get_named_params_with_correct_tied") else dict(unwrapped_model.named_parameters())
        state_dict = optimizer.state_dict()
        names = state_dict.get("names", {})

        def group_of(idx):
            param = by_name.get(names.get(idx))
            return _replica_group(param, parallel_context) if param is not None else parallel_context.dp_pg

        check_optim_state_in_sync(state_dict, parallel_context.dp_pg, group_of=group_of)
    unwrapped_model.before_optim_step_sanity_checks()


def after_optim_step_sanity_checks(config, parallel_context: ParallelContext, unwrapped_model, grad_accumulator) -> None:
    if config.general.ignore_sanity_checks:
        return
    for name, param in unwrapped_model.named_parameters():
        if param.grad is not None:
            raise AssertionError(f"Gradients of {name} should have been cleared after the optimizer step")
    unwrapped_model.after_optim_step_sanity_checks()


def check_optim_state_in_sync(optim_state_dict: dict, pg: dist.ProcessGroup, group_of=None):
    """Every optimizer state tensor is identical on the ranks of ``pg`` (or of ``group_of(state index)`` when given)."""
    for idx, st in sorted(optim_state_dict["state"].items(), key=lambda x: x[0]):
        group = group_of(idx) if group_of is not None else pg
        for name, tensor in st.items():
            if name == "step" or not isinstance(tensor, torch.Tensor):
                continue
            assert_tensor_synced_across_pg(tensor, group, msg=lambda err, name=name: f"{name} are not synced across DP {err}")
