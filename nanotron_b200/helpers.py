"""Builders used by the trainer: LR schedule, optimizer stack, throughput reporting, data-stage bookkeeping
(parity: reference src/nanotron/helpers.py:52-852)."""
from __future__ import annotations

import contextlib
import csv
import fcntl
import gc
import math
import os
import re
import time
from datetime import datetime
from functools import partial
from math import ceil
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch
from torch import nn
from torch.optim.lr_scheduler import LambdaLR
from torch.profiler import ProfilerActivity, profile, tensorboard_trace_handler

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.config import Config, DatasetStageArgs, LRSchedulerArgs, OptimizerArgs, ParallelismArgs
from nanotron_b200.logging import LogItem, human_format, log_rank
from nanotron_b200.models.base import NanotronModel
from nanotron_b200.optim.base import BaseOptimizer
from nanotron_b200.optim.fused_adamw import FusedAdamW
from nanotron_b200.optim.gradient_accumulator import FP32GradientAccumulator, GradientAccumulator
from nanotron_b200.optim.named_optimizer import NamedOptimizer
from nanotron_b200.optim.optimizer_from_gradient_accumulator import OptimizerFromGradientAccumulator
from nanotron_b200.optim.zero import ZeroDistributedOptimizer
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.random import RandomStates, get_current_random_state, get_synced_random_state
from nanotron_b200.scaling.parametrization import LearningRateForSP, LearningRateForSpectralMup, ParametrizationMethod

logger = logging.get_logger(__name__)


def _vocab_size_with_padding(orig_vocab_size: int, pg_size: int, make_vocab_size_divisible_by: int) -> int:
    """Pad the vocabulary so it divides evenly among tp ranks."""
    multiple = make_vocab_size_divisible_by * pg_size
    after = int(ceil(orig_vocab_size / multiple) * multiple)
    if after != orig_vocab_size:
        log_rank(f"[Vocab Size Padding] Padded vocab (size: {orig_vocab_size}) with {after - orig_vocab_size} dummy tokens (new size: {after})", logger=logger, level=logging.WARNING, rank=0)
    return after


def init_random_states(parallel_config: ParallelismArgs, tp_pg: dist.ProcessGroup) -> RandomStates:
    """A ``tp_synced`` state (same on all tp ranks, for dropout on replicated activations) exists only in ALL_REDUCE mode."""
    if parallel_config is None or parallel_config.tp_mode is TensorParallelLinearMode.ALL_REDUCE:
        return RandomStates({"tp_synced": get_synced_random_state(random_state=get_current_random_state(), pg=tp_pg)})
    return RandomStates({})


def lr_scheduler_builder(optimizer, lr_scheduler_args: LRSchedulerArgs, total_training_steps: int):
    """LambdaLR with warm-up (linear|constant), optional plateau until ``lr_decay_starting_step``, decay
    (linear|cosine|1-sqrt) down to ``min_decay_lr``, then constant.  One lambda per param group so groups with
    different base learning rates (muP) keep their ratio."""
    if lr_scheduler_args.lr_decay_steps is None:
        lr_decay_steps = total_training_steps
        if lr_scheduler_args.lr_warmup_steps is not None:
            lr_decay_steps -= lr_scheduler_args.lr_warmup_steps
        if lr_scheduler_args.lr_decay_starting_step is not None:
            lr_decay_steps -= lr_scheduler_args.lr_decay_starting_step
    else:
        lr_decay_steps = lr_scheduler_args.lr_decay_steps
    lr_decay_starting_step = lr_scheduler_args.lr_decay_starting_step if lr_scheduler_args.lr_decay_starting_step is not None else (lr_scheduler_args.lr_warmup_steps or 0)

    def lr_lambda(current_step: int, initial_lr: float):
        a = lr_scheduler_args
        if a.lr_warmup_steps and current_step < a.lr_warmup_steps:
            if a.lr_warmup_style == "linear":
                lmbda = initial_lr * current_step / max(a.lr_warmup_steps, 1)
            elif a.lr_warmup_style == "constant":
                lmbda = a.learning_rate
            else:
                raise ValueError(f"Unknown warmup style {a.lr_warmup_style}")
        elif current_step < lr_decay_starting_step:
            lmbda = initial_lr
        elif a.lr_decay_style is not None and current_step < lr_decay_starting_step + lr_decay_steps:
            progress = (current_step - lr_decay_starting_step) / max(lr_decay_steps, 1)
            if a.lr_decay_style == "cosine":
                lmbda = a.min_decay_lr + (initial_lr - a.min_decay_lr) * (1 + math.cos(math.pi * progress)) / 2
            elif a.lr_decay_style == "linear":
                lmbda = a.min_decay_lr + (initial_lr - a.min_decay_lr) * (1 - progress)
            elif a.lr_decay_style == "1-sqrt":
                lmbda = a.min_decay_lr + (initial_lr - a.min_decay_lr) * (1 - math.sqrt(progress))
            else:
                raise ValueError(f"Unknown decay style {a.lr_decay_style}")
        elif a.lr_decay_style is not None:
            lmbda = a.min_decay_lr
        else:
            lmbda = initial_lr
        return lmbda / initial_lr if initial_lr != 0 else 0.0

    base = optimizer.get_base_optimizer() if hasattr(optimizer, "get_base_optimizer") else optimizer
    # a resumed optimizer carries the current lr in "lr" and the base value in "initial_lr"
    lambdas = [partial(lr_lambda, initial_lr=g.get("initial_lr", g["lr"])) for g in base.param_groups]
    return LambdaLR(base, lr_lambda=lambdas)


def get_custom_weight_decay_for_named_parameters(named_parameters, model: NanotronModel, module_id_to_prefix, weight_decay: float, exclude_named_params: Optional[List[str]] = None):
    """Per-parameter weight decay: 0 for names matching any regex of ``exclude_named_params`` or listed by
    ``model.get_named_params_without_weight_decay()``."""
    named_param_groups_with_custom_weight_decay = []
    exclude_named_params = list(exclude_named_params or []) + [re.escape(n) + "$" for n in model.get_named_params_without_weight_decay()]
    for name, param in named_parameters:
        full = param.get_tied_info().get_full_name_from_module_id_to_prefix(module_id_to_prefix=module_id_to_prefix) if getattr(param, "is_tied", False) else name
        wd = 0.0 if any(re.match(pat, full) for pat in exclude_named_params) else weight_decay
        named_param_groups_with_custom_weight_decay.append({"named_params": [(name, param)], "weight_decay": wd})
    log_rank(f"[Optimizer Building] Creating {len(named_param_groups_with_custom_weight_decay)} param groups with custom weight decay", logger=logger, level=logging.DEBUG, rank=0)
    return named_param_groups_with_custom_weight_decay


def get_custom_lr_for_named_parameters(parametrization_method: ParametrizationMethod, lr: float, named_parameters, model: NanotronModel):
    """Per-parameter learning rate (base lr for standard parametrisation, fan-ratio scaled for spectral muP)."""
    assert parametrization_method in [ParametrizationMethod.SPECTRAL_MUP, ParametrizationMethod.STANDARD]
    cls = LearningRateForSpectralMup if parametrization_method == ParametrizationMethod.SPECTRAL_MUP else LearningRateForSP
    names_to_modules = dict(model.named_modules())
    mapper = cls(lr=lr, names_to_modules=names_to_modules)
    out = []
    for name, param in named_parameters:
        module_name = name.rsplit(".", 1)[0]
        out.append({"named_params": [(name, param)], "lr": mapper.get_lr(name, names_to_modules[module_name])})
    return out


def merge_named_param_groups(groups_lr, groups_wd):
    assert len(groups_lr) == len(groups_wd)
    merged: Dict[Tuple[float, float], Dict[str, Any]] = {}
    for g_lr, g_wd in zip(groups_lr, groups_wd):
        assert [n for n, _ in g_lr["named_params"]] == [n for n, _ in g_wd["named_params"]]
        key = (g_lr["lr"], g_wd["weight_decay"])
        if key not in merged:
            merged[key] = {"named_params": [], "lr": g_lr["lr"], "weight_decay": g_wd["weight_decay"]}
        merged[key]["named_params"].extend(g_lr["named_params"])
    return list(merged.values())


def init_optimizer_and_grad_accumulator(parametrization_method: ParametrizationMethod, model: nn.Module, optimizer_args: OptimizerArgs, parallel_context: ParallelContext) -> Tuple[BaseOptimizer, Optional[GradientAccumulator]]:
    """NamedOptimizer(AdamW|SGD) -> optional fp32 accumulator -> optional ZeRO-1.

    On CUDA with AdamW the base optimizer is the in-tree multi-tensor AdamW; with fp32 accumulation it also writes
    the bf16 parameters, and under ZeRO-1 gradients are reduce-scattered over dp on the flat buffer."""
    unwrapped = model.module if hasattr(model, "module") and isinstance(getattr(model, "module"), nn.Module) and not isinstance(model, NanotronModel) else model
    module_id_to_prefix = {id(m): f"{n}." if n else "" for n, m in unwrapped.named_modules()}
    module_id_to_prefix[id(unwrapped)] = ""
    named_parameters = list(unwrapped.get_named_params_with_correct_tied())
    named_parameters = [(n, p) for n, p in named_parameters if p.requires_grad]
    groups_lr = get_custom_lr_for_named_parameters(parametrization_method, optimizer_args.learning_rate_scheduler.learning_rate, named_parameters, unwrapped)
    groups_wd = get_custom_weight_decay_for_named_parameters(named_parameters, unwrapped, module_id_to_prefix, optimizer_args.weight_decay, optimizer_args.weight_decay_exclude_named_params)
    named_param_groups = merge_named_param_groups(groups_lr, groups_wd)

    def basic_optimizer_builder(named_param_groups):
        factory = optimizer_args.optimizer_factory
        if factory.name == "adamW":

            def optimizer(param_groups):
                first = param_groups[0]["params"][0] if param_groups and param_groups[0]["params"] else None
                use_native = first is not None and first.is_cuda and first.dtype == torch.float32
                if use_native or not factory.torch_adam_is_fused:
                    if use_native or first is None or first.dtype == torch.float32:
                        return FusedAdamW(param_groups, lr=optimizer_args.learning_rate_scheduler.learning_rate, weight_decay=optimizer_args.weight_decay, eps=factory.adam_eps, betas=(factory.adam_beta1, factory.adam_beta2))
                return torch.optim.AdamW(param_groups, lr=optimizer_args.learning_rate_scheduler.learning_rate, weight_decay=optimizer_args.weight_decay, eps=factory.adam_eps, betas=(factory.adam_beta1, factory.adam_beta2), fused=factory.torch_adam_is_fused and first is not None and first.is_cuda)

        elif factory.name == "sgd":

            def optimizer(param_groups):
                return torch.optim.SGD(param_groups, lr=optimizer_args.learning_rate_scheduler.learning_rate, weight_decay=optimizer_args.weight_decay)

        else:
            raise ValueError(f"Optimizer {factory.name} is not supported")
        return NamedOptimizer(named_params_or_groups=named_param_groups, optimizer_builder=optimizer)

    optimizer_builder = basic_optimizer_builder
    grad_accumulator: Optional[GradientAccumulator] = None
    dp_size = parallel_context.dp_pg.size()
    zero = optimizer_args.zero_stage > 0
    if zero and parallel_context.expert_parallel_size > 1:
        # ZeRO-1 cuts every parameter's optimizer state over the dp ranks and all-gathers the updated parameters over them; with
        # experts laid over the dp axis those ranks hold DIFFERENT experts, so the gather would stitch unrelated experts together
        raise ValueError(
            f"zero_stage={optimizer_args.zero_stage} cannot be combined with expert_parallel_size={parallel_context.expert_parallel_size}: the expert-parallel ranks "
            "are data-parallel ranks that own different experts.  Use zero_stage 0 (the optimizer state of the experts is already split over the expert-parallel ranks)."
        )
    holder: Dict[str, Any] = {}
    if optimizer_args.accumulate_grad_in_fp32:

        def grad_optimizer_builder(named_param_groups):
            def accumulator_builder(named_params_iter):
                acc = FP32GradientAccumulator(
                    named_parameters=named_parameters,
                    grad_buckets_named_params=named_parameters,
                    flat_shard_world=dp_size if zero else 1,
                )
                if zero:
                    acc.assign_param_offsets(param_name_to_offsets=holder["offsets"], dp_rank=dist.get_rank(parallel_context.dp_pg))
                holder["acc"] = acc
                return acc

            result = OptimizerFromGradientAccumulator(
                gradient_accumulator_builder=accumulator_builder,
                named_params_or_groups=named_param_groups,
                optimizer_builder=basic_optimizer_builder,
            )
            return result

        optimizer_builder = grad_optimizer_builder

    if zero:
        inner_builder = optimizer_builder

        class _Zero(ZeroDistributedOptimizer):
            pass

        def zero_builder_with_offsets(groups):
            return inner_builder(groups)

        # the accumulator needs the offsets table before it is built: compute the layout first
        from nanotron_b200.optim.flat_layout import FlatLayout

        all_named = [(n, p) for g in named_param_groups for n, p in g["named_params"]]
        holder["offsets"] = FlatLayout.build([(n, p.numel()) for n, p in all_named], world=dp_size).param_name_to_dp_rank_offsets()
        if optimizer_args.accumulate_grad_in_fp32:
            # gradient slots must follow the same order as the ZeRO layout
            named_parameters[:] = all_named
        optimizer = ZeroDistributedOptimizer(named_params_or_groups=named_param_groups, optimizer_builder=zero_builder_with_offsets, dp_pg=parallel_context.dp_pg)
        assert optimizer.param_name_to_dp_rank_offsets == holder["offsets"]
    else:
        optimizer = optimizer_builder(named_param_groups)

    if optimizer_args.accumulate_grad_in_fp32:
        grad_accumulator = holder["acc"]
        # let the fused AdamW write the bf16 parameters directly
        base = optimizer.get_base_optimizer()
        if isinstance(base, FusedAdamW):
            for name, d in grad_accumulator.parameters.items():
                s, e = grad_accumulator._master_ranges[name]
                base.set_half_target(d["fp32"], d["half"].detach().view(-1)[s:e])
    return optimizer, grad_accumulator


def get_profiler(config: Config):
    if config.profiler is not None and config.profiler.profiler_export_path is not None:
        rank0 = not dist.is_initialized() or dist.get_rank() == 0
        if not rank0:
            return contextlib.nullcontext()
        p = config.profiler
        on_trace_ready = tensorboard_trace_handler(str(p.profiler_export_path) + "/" + datetime.now().strftime("%Y%m%d-%H%M%S-" + config.general.run))
        activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        return profile(
            activities=activities,
            schedule=torch.profiler.schedule(wait=p.wait, warmup=p.warmup, active=p.active, repeat=p.repeat, skip_first=p.skip_first),
            on_trace_ready=on_trace_ready, record_shapes=p.record_shapes, profile_memory=p.profile_memory, with_stack=p.with_stack,
        )
    return contextlib.nullcontext()


def get_all_comps(n: int) -> List[List[List[int]]]:
    """Round-robin pairings of 0..n-1 (n a power of two): n-1 rounds covering every pair once."""
    assert n > 0 and (n & (n - 1)) == 0, "n must be a power of two"

    def op(l, d=4, r=1):
        assert len(l) % d == 0
        l = np.array(l).reshape(-1, d)
        l[1::2] = np.roll(l[1::2], r, axis=1)
        return l.T.reshape(-1)

    x = np.array(list(range(n)))
    comps = []
    d = 1
    while d < n:
        for r in range(d):
            comps.append(op(x, d=d, r=r).copy())
        d *= 2
    ret = np.stack(comps).reshape(len(comps), -1, 2).tolist()
    return ret


def test_all_pair_to_pair(parallel_context: ParallelContext, throughput_size: int, throughput_iters: int, only_node_to_node: bool = True):
    """Measure point-to-point bandwidth between every pair of ranks (device-timed) and log it from rank 0."""
    pg = parallel_context.world_pg
    me = dist.get_rank(pg)
    world = pg.size()
    device = parallel_context.device
    results = {}
    for a in range(world):
        for b in range(a + 1, world):
            if only_node_to_node and not (a % parallel_context.local_world_size == 0 and b % parallel_context.local_world_size == 0):
                continue
            dist.barrier(pg)
            if me in (a, b):
                t = torch.empty(throughput_size, dtype=torch.uint8, device=device)
                peer = b if me == a else a
                start = time.perf_counter()
                if device.type == "cuda":
                    torch.cuda.synchronize()
                for _ in range(throughput_iters):
                    if me == a:
                        dist.send(t, dst=peer, group=pg)
                    else:
                        dist.recv(t, src=peer, group=pg)
                if device.type == "cuda":
                    torch.cuda.synchronize()
                dt = time.perf_counter() - start
                results[(a, b)] = throughput_size * throughput_iters / dt / 1e9
                if me == a:
                    log_rank(f"[TEST] {a} -> {b}: {results[(a, b)]:.2f} GB/s", logger=logger, level=logging.WARNING)
    dist.barrier(pg)
    return results


def create_table_log(config: Config, parallel_context: ParallelContext, model_tflops, hardware_tflops, tokens_per_sec, bandwidth, num_params, slurm_job_id):
    return [
        LogItem("job_id", slurm_job_id, "s"),
        LogItem("name", config.general.run, "s"),
        LogItem("nodes", math.ceil(parallel_context.world_pg.size() / max(1, parallel_context.local_world_size)), "d"),
        LogItem("seq_len", config.tokens.sequence_length, "d"),
        LogItem("mbs", config.tokens.micro_batch_size, "d"),
        LogItem("batch_accum", config.tokens.batch_accumulation_per_replica, "d"),
        LogItem("gbs", config.global_batch_size, "d"),
        LogItem("mTFLOPs", model_tflops, ".2f"),
        LogItem("hTFLOPs", hardware_tflops, ".2f"),
        LogItem("tok/s/gpu", tokens_per_sec / parallel_context.world_pg.size(), ".2f"),
        LogItem("Mem Alloc (GB)", torch.cuda.max_memory_allocated() / 1024**3 if torch.cuda.is_available() else 0.0, ".2f"),
        LogItem("Mem Res (GB)", torch.cuda.max_memory_reserved() / 1024**3 if torch.cuda.is_available() else 0.0, ".2f"),
        LogItem("dp", config.parallelism.dp, "d"),
        LogItem("pp", config.parallelism.pp, "d"),
        LogItem("tp", config.parallelism.tp, "d"),
        LogItem("cp", config.parallelism.context_parallel_size, "d"),
        LogItem("ep", config.parallelism.expert_parallel_size, "d"),
        LogItem("pp_engine", type(config.parallelism.pp_engine).__name__, "s"),
        LogItem("tp_mode", config.parallelism.tp_mode.name, "s"),
        LogItem("tp_async_comm", str(config.parallelism.tp_linear_async_communication), "s"),
        LogItem("recompute_layer", str(config.parallelism.recompute_layer), "s"),
        LogItem("hidden_size", config.model.model_config.hidden_size, "d"),
        LogItem("hidden_act", getattr(config.model.model_config, "hidden_act", "n/a"), "s"),
        LogItem("num_layers", config.model.model_config.num_hidden_layers, "d"),
        LogItem("num_heads", config.model.model_config.num_attention_heads, "d"),
        LogItem("num_kv_heads", getattr(config.model.model_config, "num_key_value_heads", 0) or 0, "d"),
        LogItem("max_pos", config.model.model_config.max_position_embeddings, "d"),
        LogItem("vocab_size", config.model.model_config.vocab_size, "d"),
        LogItem("tie_word_embeddings", str(getattr(config.model.model_config, "tie_word_embeddings", False)), "s"),
        LogItem("dtype", str(config.model.dtype), "s"),
        LogItem("zero_stage", config.optimizer.zero_stage, "d"),
        LogItem("ddp_bucket_cap_mb", config.model.ddp_bucket_cap_mb, "d"),
        LogItem("accumulate_grad_in_fp32", str(config.optimizer.accumulate_grad_in_fp32), "s"),
        LogItem("Total Params", num_params["total"], "human_format"),
        LogItem("Local Params", num_params["local"], "human_format"),
    ]


def create_table_output(table_log: List[LogItem], column_widths: List[int]) -> str:
    def fmt(item: LogItem) -> str:
        if item.log_format == "human_format":
            return human_format(item.scalar_value)
        if item.log_format and not isinstance(item.scalar_value, str):
            return f"{item.scalar_value:{item.log_format}}"
        return str(item.scalar_value)

    header = "| " + " | ".join(i.tag.ljust(w) for i, w in zip(table_log, column_widths)) + " |"
    sep = "| " + " | ".join("-" * w for w in column_widths) + " |"
    data = "| " + " | ".join(fmt(i).ljust(w) for i, w in zip(table_log, column_widths)) + " |"
    return "\n".join([header, sep, data])


def write_to_csv(csv_filename: str, table_log: List[LogItem], model_tflops: float, slurm_job_id: str):
    """Append one row; concurrent jobs are serialised with an exclusive ``fcntl`` lock and retried."""
    os.makedirs(os.path.dirname(os.path.abspath(csv_filename)) or ".", exist_ok=True)
    header = [i.tag for i in table_log]
    row = [human_format(i.scalar_value) if i.log_format == "human_format" else (f"{i.scalar_value:{i.log_format}}" if i.log_format and not isinstance(i.scalar_value, str) else str(i.scalar_value)) for i in table_log]
    for attempt in range(10):
        try:
            exists = os.path.exists(csv_filename) and os.path.getsize(csv_filename) > 0
            with open(csv_filename, "a", newline="") as f:
                fcntl.flock(f.fileno(), fcntl.LOCK_EX | fcntl.LOCK_NB)
                try:
                    w = csv.writer(f)
                    if not exists:
                        w.writerow(header)
                    w.writerow(row)
                    f.flush()
                    os.fsync(f.fileno())
                finally:
                    fcntl.flock(f.fileno(), fcntl.LOCK_UN)
            return
        except (BlockingIOError, OSError) as e:
            log_rank(f"Attempt {attempt + 1}: could not lock {csv_filename} ({e}); retrying", logger=logger, level=logging.INFO)
            time.sleep(0.2 * (attempt + 1))
    log_rank(f"Failed to write benchmark row to {csv_filename}", logger=logger, level=logging.ERROR)


def log_throughput(config: Config, parallel_context: ParallelContext, model_tflops=0, hardware_tflops=0, tokens_per_sec=0, bandwidth=0, num_params={"total": 0, "local": 0}):
    slurm_job_id = os.environ.get("SLURM_JOB_ID", "N/A")
    table_log = create_table_log(config, parallel_context, model_tflops, hardware_tflops, tokens_per_sec, bandwidth, num_params, slurm_job_id)
    widths = [max(len(i.tag), len(str(i.scalar_value)) + 2) for i in table_log]
    log_rank(create_table_output(table_log, widths), logger=logger, level=logging.INFO, rank=0)
    if dist.get_rank(parallel_context.world_pg) == 0 and config.general.benchmark_csv_path is not None:
        write_to_csv(str(config.general.benchmark_csv_path), table_log, model_tflops, slurm_job_id)


def compute_remain_train_steps_of_a_data_stage_from_ckp(stage: DatasetStageArgs, config: Config, metadata) -> int:
    def is_last_stage():
        return stage == sorted(config.data_stages, key=lambda x: x.start_training_step)[-1]

    def is_resume_from_training():
        return metadata.last_train_step > 0

    if is_last_stage():
        total = config.tokens.train_steps
    else:
        stages = sorted(config.data_stages, key=lambda x: x.start_training_step)
        nxt = next((s for s in stages if s.start_training_step > stage.start_training_step), None)
        total = nxt.start_training_step
    last_train_steps = metadata.last_train_step if is_resume_from_training() else stage.start_training_step
    return total - last_train_steps


def get_consumed_train_samples_of_a_data_stage_from_ckp(stage: DatasetStageArgs, metadata) -> Optional[int]:
    start = next((s.consumed_train_samples for s in metadata.data_stages if s.start_training_step == stage.start_training_step), None)
    return start
