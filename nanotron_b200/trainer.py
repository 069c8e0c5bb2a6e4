"""``DistributedTrainer``: builds everything from a ``Config`` and runs the training loop
(parity: reference src/nanotron/trainer.py:131-1415; same constructor, hooks and checkpoint behaviour).

Data parallelism does not wrap the model in ``DistributedDataParallel``: gradients live in one flat fp32 buffer
(see ``optim.gradient_accumulator``) that is reduced with a single collective after the last micro-batch
(reduce-scatter under ZeRO-1, all-reduce otherwise); without fp32 accumulation the parameter gradients are
all-reduced coalesced.  Throughput is timed with CUDA events and reported as the max over ranks.
"""
from __future__ import annotations

import datetime
import gc
import json
import os
import shutil
import signal
import time
from dataclasses import asdict
from pathlib import Path
from pprint import pformat
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple, Type, Union, cast

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.config import Config, DatasetStageArgs, ExistingCheckpointInit, ParallelismArgs, RandomInit, SpectralMupInit, get_config_from_file
from nanotron_b200.constants import LATEST_FILE_NAME, MODEL_CONFIG_FILE_NAME
from nanotron_b200.helpers import (
    _vocab_size_with_padding,
    compute_remain_train_steps_of_a_data_stage_from_ckp,
    get_consumed_train_samples_of_a_data_stage_from_ckp,
    get_profiler,
    init_optimizer_and_grad_accumulator,
    init_random_states,
    log_throughput,
    lr_scheduler_builder,
)
from nanotron_b200.logging import LoggerWriter, LogItem, human_format, log_libraries_versions, log_memory, log_rank, nanotron_timer, set_ranks_logging_level
from nanotron_b200.models.base import NanotronModel, build_model, check_model_has_grad
from nanotron_b200.optim.clip_grads import clip_grad_norm
from nanotron_b200.optim.zero import ZeroDistributedOptimizer
from nanotron_b200.parallel import ParallelContext
from nanotron_b200.parallel.parameters import NanotronParameter, sanity_check
from nanotron_b200.parallel.pipeline_parallel.engine import PipelineEngine
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer
from nanotron_b200.parallel.pipeline_parallel.utils import get_pp_rank_of
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode
from nanotron_b200.parallel.tensor_parallel.nn import TensorParallelRowLinear
from nanotron_b200.parallel.tied_parameters import create_pg_for_tied_weights, get_tied_id_to_param, sync_tied_weights_gradients, tie_parameters
from nanotron_b200.random import set_random_seed
from nanotron_b200.utils import annotate
from nanotron_b200.sanity_checks import after_optim_step_sanity_checks, after_tbi_sanity_checks, before_optim_step_sanity_checks, before_tbi_sanity_checks
from nanotron_b200.scaling.parametrization import ParametrizationMethod
from nanotron_b200.serialize import load_lr_scheduler, load_meta, load_optimizer, load_weights, parse_ckpt_path, save, save_random_states
from nanotron_b200.serialize.metadata import DataStageMetadata, TrainingMetadata

logger = logging.get_logger(__name__)


def _model_registry():
    from nanotron_b200.models.llama import LlamaForTraining
    from nanotron_b200.models.qwen import Qwen2ForTraining
    from nanotron_b200.models.starcoder2 import Starcoder2ForTraining

    return {"LlamaConfig": LlamaForTraining, "Qwen2Config": Qwen2ForTraining, "Starcoder2Config": Starcoder2ForTraining}


class _Registry(dict):
    def __missing__(self, key):
        reg = _model_registry()
        self.update(reg)
        if key in reg:
            return reg[key]
        raise KeyError(key)

    def __contains__(self, key):
        return key in _model_registry() or dict.__contains__(self, key)


CONFIG_TO_MODEL_CLASS = _Registry()


class DistributedTrainer:
    def __init__(
        self,
        config_or_config_file: Union[Config, str],
        config_class: Type[Config] = Config,
        model_config_class: Optional[Type] = None,
        model_class: Optional[Type[NanotronModel]] = None,
    ):
        super().__init__()
        self.config = config_or_config_file if isinstance(config_or_config_file, Config) else get_config_from_file(config_or_config_file, config_class=config_class, model_config_class=model_config_class)
        self.model_config = self.config.model.model_config
        if model_class is not None:
            CONFIG_TO_MODEL_CLASS[self.model_config.__class__.__name__] = model_class
        par = self.config.parallelism
        self.parallel_context = ParallelContext(
            tensor_parallel_size=par.tp, pipeline_parallel_size=par.pp, data_parallel_size=par.dp,
            expert_parallel_size=par.expert_parallel_size, context_parallel_size=par.context_parallel_size,
        )
        if self.config.kernels is not None:
            from nanotron_b200 import ops

            ops.set_mode("torch" if self.config.kernels.ops == "torch" else "auto")
            if self.config.kernels.gemm in ("auto", "cublas", "tcgen05"):
                ops.set_gemm(self.config.kernels.gemm)
            if self.config.kernels.attention in ("auto", "native", "sdpa"):
                ops.set_attention(self.config.kernels.attention)
            if getattr(self.config.kernels, "linear", "bf16") in ("bf16", "fp8"):
                ops.set_linear(self.config.kernels.linear)
        self.pre_init()
        if self.config.logging is None:
            from nanotron_b200.config import LoggingArgs

            self.config.logging = LoggingArgs()
        set_ranks_logging_level(parallel_context=self.parallel_context, logging_config=self.config.logging)
        log_libraries_versions(logger=logger)
        log_rank("Config:\n" + pformat(self.config), logger=logger, level=logging.DEBUG, rank=0)
        # the named random states (tp_synced) are drawn from the configured seed on every rank ...
        set_random_seed(self.config.general.seed)
        self.random_states = init_random_states(parallel_config=par, tp_pg=self.parallel_context.tp_pg)
        # ... while the default generator differs per tp / pp rank so that sharded weights are not initialised identically
        set_random_seed(self.config.general.seed + dist.get_rank(self.parallel_context.tp_pg) + 1000 * dist.get_rank(self.parallel_context.pp_pg))
        self.model = self.init_model()
        self.unwrapped_model: NanotronModel = self.model
        if dist.get_rank(self.parallel_context.world_pg) in self.logger_ranks and dist.get_rank(self.parallel_context.world_pg) != 0:
            # the metric line of every step is printed by the rank that holds the loss (the last pipeline stage): that line follows
            # ``log_level`` like the rest of the run's console output, not ``log_level_replica``
            from nanotron_b200.logging.base import show_metric_lines

            show_metric_lines(self.config.logging.log_level or "info")
        self._configure_pipeline_p2p()
        parametrization_method = ParametrizationMethod.SPECTRAL_MUP if hasattr(self.config.model.init_method, "use_mup") else ParametrizationMethod.STANDARD
        symm_alloc = self._maybe_enable_symmetric_buffers()
        try:
            self.optimizer, self.grad_accumulator = init_optimizer_and_grad_accumulator(parametrization_method=parametrization_method, model=self.model, optimizer_args=self.config.optimizer, parallel_context=self.parallel_context)
        finally:
            from nanotron_b200.optim.flat_layout import set_buffer_allocator

            set_buffer_allocator(None)
        self.fused_dp = None
        if symm_alloc is not None:
            from nanotron_b200.optim.fused_adamw import FusedAdamW
            from nanotron_b200.optim.fused_zero import FusedDataParallelStep

            if isinstance(self.optimizer.get_base_optimizer(), FusedAdamW) and self.grad_accumulator is not None:
                self.fused_dp = FusedDataParallelStep(symm_alloc, self.grad_accumulator, self.optimizer, self.parallel_context.dp_pg, self.parallel_context.mp_pg, self.config.optimizer.clip_grad)
                self.fused_dp.exclude_tied_duplicates(self.unwrapped_model.get_named_params_with_correct_tied(), dist.get_rank(self.parallel_context.world_pg))
                if self.config.optimizer.overlap_grad_reduce:
                    early = self.fused_dp.install_overlap(self.unwrapped_model, list(self.unwrapped_model.get_named_params_with_correct_tied()))
                    # the pipeline engines enter this context around the last micro-batch's backward
                    self.grad_accumulator.prepare_last_backward = self.fused_dp.prepare_last_backward
                    log_rank(f"Gradient reduce-scatter overlapped with the last backward: {early} buckets", logger=logger, level=logging.INFO, rank=0)
                log_rank("Data-parallel step: in-kernel NVLink reduce-scatter + AdamW + all-gather", logger=logger, level=logging.INFO, rank=0)
        if self.init_checkpoint_path is not None and self.config.checkpoints.load_optimizer:
            load_optimizer(optimizer=self.optimizer, parallel_context=self.parallel_context, root_folder=self.init_checkpoint_path, param_shard_metadata=self.param_shard_metadata, model=self.unwrapped_model, map_location="cpu")
        self.lr_scheduler = lr_scheduler_builder(optimizer=self.optimizer, lr_scheduler_args=self.config.optimizer.learning_rate_scheduler, total_training_steps=self.config.tokens.train_steps)
        if self.init_checkpoint_path is not None and self.config.checkpoints.load_lr_scheduler:
            load_lr_scheduler(lr_scheduler=self.lr_scheduler, is_zero=self.config.optimizer.zero_stage, parallel_context=self.parallel_context, root_folder=self.init_checkpoint_path)
        if self.init_checkpoint_path is not None and self.config.checkpoints.load_optimizer:
            ckpt_meta = load_meta(parallel_context=self.parallel_context, root_folder=self.init_checkpoint_path)
            self.metadata: TrainingMetadata = ckpt_meta.metas
            assert isinstance(self.metadata, TrainingMetadata)
            log_rank(str(self.metadata), logger=logger, level=logging.INFO, rank=0)
        else:
            stages = [DataStageMetadata(name=s.name, start_training_step=s.start_training_step, consumed_train_samples=0, sequence_length=s.sequence_length or self.config.tokens.sequence_length) for s in (self.config.data_stages or [])]
            self.metadata = TrainingMetadata(consumed_train_samples=0, consumed_tokens_total=0, last_train_step=0, last_stage_idx=0 if stages else None, data_stages=stages or None)
        self.micro_batch_size = self.config.tokens.micro_batch_size
        self.n_micro_batches_per_batch = self.config.tokens.batch_accumulation_per_replica
        self.global_batch_size = self.micro_batch_size * self.n_micro_batches_per_batch * self.parallel_context.dp_pg.size()
        self.sequence_length = self.config.tokens.sequence_length
        self.iteration_step = self.metadata.last_train_step
        self.limit_val_batches = self.config.tokens.limit_val_batches
        self.current_dataloader: Optional[Iterator] = None
        self.current_base_dl = None
        self._stop_requested = False
        self._kill_switch_path = Path(os.environ["NANOTRON_KILL_SWITCH"]) if os.environ.get("NANOTRON_KILL_SWITCH") else None
        from nanotron_b200.metrics_logging import MetricsLogger

        self.metrics_logging = MetricsLogger(self.config)
        self._detailed_metrics: Optional[Dict[str, float]] = None
        # NANOTRON_METRICS_JSONL=<file>: every logged step is also appended there as one JSON object (works without wandb)
        self._metrics_jsonl = os.environ.get("NANOTRON_METRICS_JSONL")
        self.post_init()

    def _pipeline_p2ps(self):
        from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

        seen = {}
        for m in self.unwrapped_model.modules():
            if isinstance(m, PipelineBlock):
                seen[id(m.p2p)] = m.p2p
        return list(seen.values())

    def _configure_pipeline_p2p(self):
        """Micro-batches of a data stage all have the same geometry: let pipeline stages learn the shapes they exchange during the
        first micro-batch and send bare payloads afterwards (``pp_static_shapes``)."""
        if self.parallel_context.pp_pg.size() == 1:
            return
        for p2p in self._pipeline_p2ps():
            p2p.expect_static(bool(getattr(self.config.parallelism, "pp_static_shapes", True)))

    def _maybe_enable_symmetric_buffers(self):
        """Put the flat gradient / parameter buffers in peer-mapped memory when the fused data-parallel step applies."""
        ctx, opt = self.parallel_context, self.config.optimizer
        if opt.fused_zero_comm is False or ctx.device.type != "cuda" or ctx.dp_pg.size() == 1:
            return None
        if not opt.accumulate_grad_in_fp32 or opt.optimizer_factory.name != "adamW" or ctx.cp_pg.size() > 1 or ctx.expert_parallel_size > 1:
            return None
        if ctx.world_size > ctx.local_world_size:
            dp_ranks = dist.get_global_ranks(ctx.dp_pg)
            if len({r // ctx.local_world_size for r in dp_ranks}) > 1:
                return None  # the dp group spans nodes: NVLink peer access does not reach
        from nanotron_b200 import ops
        from nanotron_b200.optim.flat_layout import set_buffer_allocator
        from nanotron_b200.parallel import symm

        if ops.get_mode() == "torch" or not symm.is_available(ctx.dp_pg):
            return None
        alloc = symm.SymmetricAllocator(ctx.dp_pg)
        set_buffer_allocator(lambda numel, dtype, device: alloc.zeros(numel, dtype).tensor)
        return alloc

    # ------------------------------------------------------------------ hooks
    def pre_init(self):
        self.init_checkpoint_path = parse_ckpt_path(config=self.config, parallel_context=self.parallel_context)
        self.param_shard_metadata = None

    def post_init(self):
        self.s3_mover = None
        if self.config.s3_upload is not None:
            from nanotron_b200.s3_checkpoints import S3Mover

            self.s3_mover = S3Mover(
                local_path=str(self.config.checkpoints.checkpoints_path), s3_path=str(self.config.s3_upload.upload_s3_path),
                remove_after_upload=self.config.s3_upload.remove_after_upload, s5cmd_numworkers=self.config.s3_upload.s5cmd_numworkers,
                s5cmd_concurrency=self.config.s3_upload.s5cmd_concurrency, s5cmd_path=self.config.s3_upload.s5cmd_path,
                dummy=bool(int(os.environ.get("LOCAL_RANK", "0")) != 0),
            )

    def pre_training(self, *args, **kwargs):
        self._install_signal_handlers()
        metadata = self.metadata
        log_rank(f"Start training] datetime: {datetime.datetime.now()} | layout: {self.config.parallelism.describe()} | mbs: {self.micro_batch_size} | grad_accum: {self.n_micro_batches_per_batch} | global_batch_size: {self.global_batch_size} | sequence_length: {self.sequence_length} | train_steps: {self.config.tokens.train_steps} | start_iteration_step: {metadata.last_train_step} | consumed_train_samples: {metadata.consumed_train_samples}", logger=logger, level=logging.INFO, rank=0)
        self._wandb = None
        is_logger = dist.get_rank(self.parallel_context.world_pg) == self.logger_ranks[0]
        per_tp_runs = self._shard_suffix() != "" and self._is_metrics_rank()
        if os.environ.get("WANDB_MODE", "disabled") != "disabled" and (is_logger or per_tp_runs):
            try:
                import wandb

                self._wandb = wandb
                # with detailed metrics every model shard (tp rank, pp stage) has a run of its own, grouped under the run name
                name = f"{self.config.general.run}" + (f"_{self._shard_suffix()}" if per_tp_runs else "")
                wandb.init(project=self.config.general.project, name=name, group=self.config.general.run if per_tp_runs else None, config={"nanotron_config": self.config.as_dict()})
            except ImportError:
                self._wandb = None

    def post_train_step(self):
        if self.s3_mover is not None:
            self.s3_mover.update()

    def post_training(self):
        if self.s3_mover is not None:
            self.s3_mover.distributed_wait_for_completion(group=self.parallel_context.world_pg)

    def _install_signal_handlers(self):
        """SIGTERM / SIGUSR1 request a clean stop: the loop saves a checkpoint at the next step boundary and exits."""

        def handler(signum, frame):
            self._stop_requested = True

        try:
            signal.signal(signal.SIGTERM, handler)
            signal.signal(signal.SIGUSR1, handler)
        except ValueError:
            pass  # not the main thread

    def _should_stop(self) -> bool:
        """True on every rank when any rank was signalled or the kill-switch file exists (decided collectively)."""
        flag = self._stop_requested or (self._kill_switch_path is not None and self._kill_switch_path.exists())
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=self.parallel_context.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.parallel_context.world_pg)
        return bool(t.item())

    # ------------------------------------------------------------------ data stages
    def _update_dataloader_based_on_training_stages(self, dataloaders):
        if not isinstance(dataloaders, dict):
            if self.current_dataloader is None:
                self.current_base_dl = dataloaders
                self.current_dataloader = self._wrap(dataloaders)
            return
        assert len(dataloaders) > 0, "No dataloaders provided"
        stages = self.config.data_stages

        def find_stage_idx_to_resume():
            reversed_stages = sorted(stages, key=lambda s: s.start_training_step, reverse=True)
            for idx, stage in enumerate(reversed_stages):
                if self.iteration_step >= stage.start_training_step:
                    return len(stages) - idx - 1
            return None

        stage_idx_to_resume = find_stage_idx_to_resume()
        for stage_idx, stage in enumerate(stages):
            if stage_idx < (self.metadata.last_stage_idx or 0):
                continue
            is_resume = self.current_dataloader is None and stage_idx_to_resume == stage_idx
            if (stage.start_training_step == self.iteration_step) or is_resume:
                if self.current_dataloader is not None:
                    prev = stages[stage_idx - 1].name
                    self.current_base_dl = None
                    self.current_dataloader = None
                    gc.collect()
                    log_rank(f"[Training Stage: {prev}] finished; clearing its dataloader", logger=logger, level=logging.INFO, rank=0)
                self.metadata.last_stage_idx = stage_idx
                if not is_resume:
                    remaining = compute_remain_train_steps_of_a_data_stage_from_ckp(stage, self.config, self.metadata)
                    log_rank(f"[Training Plan] Stage {stage.name} has {remaining} remaining training steps and has consumed {get_consumed_train_samples_of_a_data_stage_from_ckp(stage, self.metadata)} samples", logger=logger, level=logging.INFO, rank=0)
                dl = dataloaders[stage.name]
                dl = dl() if callable(dl) else dl
                self.current_base_dl = dl
                self.current_dataloader = self._wrap(dl)
                new_len = stage.sequence_length or self.config.tokens.sequence_length
                if new_len != self.sequence_length and self.parallel_context.pp_pg.size() > 1:
                    for p2p in self._pipeline_p2ps():
                        p2p.reset_static()  # every rank switches stage at the same step: the next micro-batch re-learns the shapes
                self.sequence_length = new_len
                break
        assert self.current_dataloader is not None, "no data stage applies to the current step"

    def _wrap(self, dl):
        from nanotron_b200.data.dataloader import sanity_check_dataloader

        return sanity_check_dataloader(dataloader=iter(dl) if not hasattr(dl, "__next__") else dl, parallel_context=self.parallel_context, config=self.config)

    # ------------------------------------------------------------------ loop
    def train(self, dataloader_or_dls, **kwargs) -> None:
        self.pre_training(**kwargs)
        if self.config.checkpoints is not None and self.config.checkpoints.save_initial_state and self.init_checkpoint_path is None:
            self.save_checkpoint()
        self.pipeline_engine: PipelineEngine = self.config.parallelism.pp_engine
        self.pipeline_engine.nb_microbatches = self.n_micro_batches_per_batch
        log_memory(logger=logger)
        self.initial_iter_step = self.metadata.last_train_step + 1
        self.last_iter_step = self.config.tokens.train_steps
        prof = get_profiler(config=self.config)
        from nanotron_b200 import fault_tolerance

        world_rank = dist.get_rank(self.parallel_context.world_pg)
        self.heartbeat, self.watchdog = fault_tolerance.from_env(world_rank, self.parallel_context.world_pg.size())
        step_deadline = float(os.environ["NANOTRON_STEP_DEADLINE"]) if os.environ.get("NANOTRON_STEP_DEADLINE") else None
        try:
            self._train_loop(prof, dataloader_or_dls, step_deadline)
        except BaseException:
            if self.heartbeat is not None:
                self.heartbeat.stop("failed")  # peers learn of the failure from the heartbeat before their next launch
            raise
        if self.heartbeat is not None:
            self.heartbeat.stop("done")
        dist.barrier(self.parallel_context.world_pg)
        if self.config.checkpoints is not None and self.config.checkpoints.save_final_state and not self._stop_requested:
            if self.iteration_step % self.config.checkpoints.checkpoint_interval != 0:
                self.save_checkpoint()
        self.post_training()

    def _train_loop(self, prof, dataloader_or_dls, step_deadline):
        from nanotron_b200 import fault_tolerance

        with prof:
            for self.iteration_step in range(self.initial_iter_step, self.last_iter_step + 1):
                if hasattr(prof, "step"):
                    prof.step()
                if self.watchdog is not None:
                    self.watchdog.raise_if_failed()  # between steps: nothing of ours is in flight towards a dead peer
                if self.heartbeat is not None:
                    self.heartbeat.beat(self.iteration_step)
                self.iteration_timer = nanotron_timer("iteration_time", "cuda" if self.parallel_context.device.type == "cuda" else "cpu", cuda_sync=False, enabled=True)
                self.iteration_timer.start()
                self._update_dataloader_based_on_training_stages(dataloader_or_dls)
                with fault_tolerance.StepDeadline(step_deadline):
                    outputs, loss_avg, z_loss_avg = self.training_step(dataloader=self.current_dataloader)
                # bookkeeping
                self.metadata.consumed_train_samples += self.global_batch_size
                self.metadata.consumed_tokens_total = (self.metadata.consumed_tokens_total or 0) + self.global_batch_size * self.sequence_length
                self.metadata.last_train_step = self.iteration_step
                if self.metadata.data_stages:
                    stage = self.metadata.data_stages[self.metadata.last_stage_idx]
                    stage.consumed_train_samples += self.global_batch_size
                    base = self.current_base_dl
                    ds = getattr(base, "dataset", None)
                    if ds is not None and hasattr(ds, "update_consumption_metrics"):
                        # blended token files: account this step's global batch (a range of the blend index) to its folders
                        ds.update_consumption_metrics(start_idx=stage.consumed_train_samples - self.global_batch_size, end_idx=stage.consumed_train_samples, sequence_length=self.sequence_length)
                    if ds is not None and hasattr(ds, "get_consumption_stats"):
                        import inspect

                        if "consumed_samples" in inspect.signature(ds.get_consumption_stats).parameters:
                            stats = ds.get_consumption_stats(consumed_samples=stage.consumed_train_samples)  # job-wide, from the sample index
                        else:
                            stats = ds.get_consumption_stats()
                        for folder, s in stats.items():
                            stage.consumed_tokens_per_dataset_folder[folder] = s["tokens"]
                if (self.iteration_step - 1) % self.config.logging.iteration_step_info_interval == 0:
                    self.train_step_logs(outputs=outputs, loss_avg=loss_avg, z_loss_avg=z_loss_avg)
                if self._detailed_metrics is not None:  # a detailed-metrics step that is not a console step
                    self._emit_metrics([LogItem(k, v, "human_format") for k, v in self._detailed_metrics.items()])
                    self._detailed_metrics = None
                stop = (self._kill_switch_path is not None or self._stop_requested) and self._should_stop()
                if self.config.checkpoints is not None and (self.iteration_step % self.config.checkpoints.checkpoint_interval == 0 or stop):
                    self.save_checkpoint()
                if stop:
                    log_rank("Stop requested (signal or kill-switch file): checkpoint saved, leaving the training loop", logger=logger, level=logging.WARNING, rank=0)
                    break

    def prepare_training(self):
        """Set up what ``train`` sets up before its loop, for callers that drive ``training_step`` themselves."""
        self.pipeline_engine: PipelineEngine = self.config.parallelism.pp_engine
        self.pipeline_engine.nb_microbatches = self.n_micro_batches_per_batch
        self.initial_iter_step = self.metadata.last_train_step + 1
        self.iteration_step = self.initial_iter_step

    def training_step(self, dataloader: Iterator[Dict[str, Union[torch.Tensor, TensorPointer]]]):
        if hasattr(self.unwrapped_model, "clear_all_tbi_logs"):
            self.unwrapped_model.clear_all_tbi_logs()  # what the modules recorded during the previous step stays readable until here
        before_tbi_sanity_checks(self.config, self.parallel_context, self.unwrapped_model, self.grad_accumulator, self.lr_scheduler)
        if self.iteration_step < self.initial_iter_step + 5:
            log_memory(logger=logger)
        with nanotron_timer("train_batch_iter"), annotate("train_batch_iter"):
            outputs = self.pipeline_engine.train_batch_iter(
                model=self.model, pg=self.parallel_context.pp_pg, batch=(next(dataloader) for _ in range(self.n_micro_batches_per_batch)),
                nb_microbatches=self.n_micro_batches_per_batch, grad_accumulator=self.grad_accumulator,
            )
        after_tbi_sanity_checks(self.config, self.parallel_context, self.unwrapped_model, self.grad_accumulator)
        fused = self.fused_dp is not None
        # tied / replicated-by-design parameters (norm weights under sequence parallelism, tied embeddings).  This sum runs BEFORE the
        # data-parallel reduction: under ZeRO-1 that reduction is an in-place reduce-scatter after which only this rank's flat shard is
        # valid, and two pipeline stages that tie a parameter own different slices of it.  Both reductions are linear, so the order
        # does not change the result (the reference all-reduces whole gradients over dp first, trainer.py:643-661).
        sync_tied_weights_gradients(module=self.unwrapped_model, parallel_context=self.parallel_context, grad_accumulator=self.grad_accumulator)
        if not fused:
            with nanotron_timer("sync_gradients"), annotate("sync_gradients"):
                self._sync_gradients()
        self.grad_norm_unclipped = None
        if self.config.optimizer.clip_grad is not None and not fused:
            with nanotron_timer("clip_gradients"), annotate("clip_gradients"):
                self.grad_norm_unclipped = self._clip_gradients()
        # loss average over data (and context) parallel replicas, for logging
        loss_avg = z_loss_avg = None
        if isinstance(outputs[0]["loss"], torch.Tensor):
            loss_avg = torch.stack([o["loss"] for o in outputs]).sum()
            z = [o["z_loss"] for o in outputs if "z_loss" in o and isinstance(o["z_loss"], torch.Tensor)]
            z_loss_avg = torch.stack(z).sum() if z else None
            vals = loss_avg if z_loss_avg is None else torch.stack([loss_avg, z_loss_avg])
            pg = self.parallel_context.dp_cp_pg
            if pg.size() > 1:
                dist.all_reduce(vals, group=pg, op=dist.ReduceOp.SUM)
                vals = vals / pg.size()
            loss_avg, z_loss_avg = (vals, None) if z_loss_avg is None else (vals[0], vals[1])
        # optimizer states loaded on CPU are moved to the device right before the first step
        if self.init_checkpoint_path is not None and self.config.checkpoints.load_optimizer and self.iteration_step == self.initial_iter_step:
            self._move_optimizer_state_to_device()
        before_optim_step_sanity_checks(self.config, self.parallel_context, self.unwrapped_model, self.grad_accumulator, self.optimizer)
        self._detailed_metrics = None
        if self.metrics_logging.log_level > 0 and self.iteration_step % self.metrics_logging.log_detail_interval == 0 and self._is_metrics_rank():
            # per-layer statistics of weights and of the gradients this step applies (after clipping, before they are cleared)
            with torch.no_grad():
                # gradient statistics only where this rank holds whole reduced gradients (a sharded exchange leaves it one slice)
                sliced = fused or (self.config.optimizer.zero_stage > 0 and self.parallel_context.dp_pg.size() > 1)
                collected = self.metrics_logging.collect_all_metrics(model=self.unwrapped_model, grad_accumulator=None if sliced else self.grad_accumulator, iteration_step=self.iteration_step)
            self._detailed_metrics = {k: float(v) for k, v in collected.items()}
        with nanotron_timer("optimizer_step"), annotate("optimizer_step"):
            if fused:
                self.grad_norm_unclipped = self.fused_dp.step()
            else:
                self.optimizer.step()
            self.optimizer.zero_grad()
        from nanotron_b200 import ops

        if ops.get_linear() == "fp8":
            from nanotron_b200.fp8 import weight_cache

            weight_cache.invalidate()  # the weights moved: their quantised copies are recomputed on first use
        self.lr_scheduler.step()
        after_optim_step_sanity_checks(self.config, self.parallel_context, self.unwrapped_model, self.grad_accumulator)
        self.post_train_step()
        return outputs, loss_avg, z_loss_avg

    def _param_is_expert(self, p) -> bool:
        return isinstance(p, NanotronParameter) and p.is_sharded and p.get_sharded_info().is_expert_sharded(self.parallel_context)

    def _sync_gradients(self):
        """Average gradients over the data-parallel (x context-parallel) replicas."""
        ctx = self.parallel_context
        zero = self.optimizer.inherit_from(ZeroDistributedOptimizer)
        ep = ctx.expert_parallel_size
        if ep > 1:
            self._sync_gradients_with_experts()
            return
        if ctx.dp_cp_pg.size() == 1:
            return
        if self.grad_accumulator is not None:
            if zero:
                if ctx.cp_pg.size() > 1:
                    self.grad_accumulator.sync_gradients_across_dp(ctx.cp_pg, dist.ReduceOp.AVG, reduce_scatter=False)
                self.grad_accumulator.sync_gradients_across_dp(ctx.dp_pg, dist.ReduceOp.AVG, reduce_scatter=True)
            else:
                self.grad_accumulator.sync_gradients_across_dp(ctx.dp_cp_pg, dist.ReduceOp.AVG, reduce_scatter=False)
            return
        from nanotron_b200.parallel.data_parallel import sync_gradients_across_dp

        sync_gradients_across_dp(self.unwrapped_model, ctx.dp_cp_pg, reduce_op=dist.ReduceOp.AVG)

    def _sync_gradients_with_experts(self):
        """Expert weights are replicated over ``expert_dp`` only and saw tokens of all ``ep`` ranks: their gradients
        are averaged over expert_dp (x cp) and divided by ep; everything else is averaged over dp x cp."""
        ctx = self.parallel_context
        dense, experts = [], []
        for name, p in self.unwrapped_model.get_named_params_with_correct_tied():
            if not p.requires_grad:
                continue
            g = self.grad_accumulator.get_grad_buffer(name) if self.grad_accumulator is not None else p.grad
            if g is None:
                continue
            (experts if self._param_is_expert(p) else dense).append(g)
        from nanotron_b200.parallel.expert_parallel import sync_dense_and_expert_gradients

        sync_dense_and_expert_gradients(dense, experts, ctx)

    def _clip_gradients_fused(self):
        """CUDA fast path: one flat sum-of-squares kernel over the fp32 gradient buffer (this rank's shard under
        ZeRO-1), reduced over model-parallel (and dp when sharded) groups; the clip coefficient stays on the device
        and is applied inside the AdamW kernel instead of a separate pass over all gradients."""
        from nanotron_b200.ops import native
        from nanotron_b200.optim.fused_adamw import FusedAdamW

        ctx = self.parallel_context
        acc = self.grad_accumulator
        zero = self.optimizer.inherit_from(ZeroDistributedOptimizer)
        buf = acc._contiguous_fp32_grad_buffer
        if zero and ctx.dp_pg.size() > 1:
            s, e = acc.flat_shard_range
            view = buf[s:e]
        else:
            view = buf
        total = native.sumsq(view)
        # tied parameters are counted once: ranks other than the first of a tie group remove their copy
        world_rank = dist.get_rank(ctx.world_pg)
        me = dist.get_rank(ctx.dp_pg)
        for n, p in self.unwrapped_model.get_named_params_with_correct_tied():
            if not (p.requires_grad and p.is_tied):
                continue
            ranks = sorted(p.get_tied_info().global_ranks)
            if len(ranks) > 1 and world_rank != ranks[0]:
                g = acc.get_grad_buffer(n).view(-1)
                if zero and ctx.dp_pg.size() > 1:
                    rng = self.optimizer.param_name_to_dp_rank_offsets[n].get(me)
                    if rng is None:
                        continue
                    g = g[rng[0] : rng[1]]
                total = total - g.float().pow(2).sum()
        dist.all_reduce(total, group=ctx.mp_pg, op=dist.ReduceOp.SUM)
        if zero and ctx.dp_pg.size() > 1:
            dist.all_reduce(total, group=ctx.dp_pg, op=dist.ReduceOp.SUM)
        norm = total.sqrt()
        coef = torch.clamp(self.config.optimizer.clip_grad / (norm + 1e-6), max=1.0)
        self.optimizer.get_base_optimizer().grad_scale = coef
        return norm.squeeze()

    def _can_fuse_clip(self) -> bool:
        from nanotron_b200 import ops
        from nanotron_b200.optim.fused_adamw import FusedAdamW

        return (
            self.grad_accumulator is not None and self.parallel_context.device.type == "cuda" and ops.get_mode() != "torch"
            and isinstance(self.optimizer.get_base_optimizer(), FusedAdamW) and self.parallel_context.expert_parallel_size == 1
            and not self.optimizer.get_base_optimizer()._flat_failed
        )

    def _clip_gradients(self):
        ctx = self.parallel_context
        zero = self.optimizer.inherit_from(ZeroDistributedOptimizer)
        if self._can_fuse_clip():
            return self._clip_gradients_fused()
        named = [(n, p) for n, p in self.unwrapped_model.get_named_params_with_correct_tied() if p.requires_grad]
        if zero and self.grad_accumulator is not None and ctx.dp_pg.size() > 1:
            # gradients are only valid on this rank's shard: norm over the owned slices, summed over dp as well
            me = dist.get_rank(ctx.dp_pg)
            world_rank = dist.get_rank(ctx.world_pg)
            slices, owned = [], []
            for n, p in named:
                rng = self.optimizer.param_name_to_dp_rank_offsets[n].get(me) if hasattr(self.optimizer, "param_name_to_dp_rank_offsets") else None
                if rng is None:
                    continue
                piece = self.grad_accumulator.get_grad_buffer(n).view(-1)[rng[0] : rng[1]]
                owned.append(piece)  # every owned slice is scaled ...
                if p.is_tied:
                    ranks = p.get_tied_info().global_ranks
                    # ... but a tied parameter is counted in the norm by the first rank of its tie group only (same dp rank by construction)
                    if ctx.get_local_ranks(world_rank)["dp"] == me and world_rank != sorted(ranks)[0] and len(ranks) > 1:
                        continue
                slices.append(piece)
            return clip_grad_norm(mp_pg=ctx.mp_pg, named_parameters=named, grad_accumulator=self.grad_accumulator, max_norm=self.config.optimizer.clip_grad, extra_reduce_group=ctx.dp_pg,
                                  grad_slices=slices, scale_slices=owned)
        extra = ctx.ep_pg if ctx.expert_parallel_size > 1 else None
        if extra is not None:
            # dense params are replicated over ep: count them on ep rank 0 only so the ep-sum is exact
            me_ep = dist.get_rank(ctx.ep_pg)
            grads = []
            world_rank = dist.get_rank(ctx.world_pg)
            for n, p in named:
                if not self._param_is_expert(p) and me_ep != 0:
                    continue
                if p.is_tied and world_rank != sorted(p.get_tied_info().global_ranks)[0]:
                    continue
                g = self.grad_accumulator.get_grad_buffer(n) if self.grad_accumulator is not None else p.grad
                if g is not None:
                    grads.append(g)
            total = clip_grad_norm(mp_pg=ctx.mp_pg, named_parameters=named, grad_accumulator=self.grad_accumulator, max_norm=float("inf"), extra_reduce_group=extra, grad_slices=grads)
            coef = torch.clamp(self.config.optimizer.clip_grad / (total + 1e-6), max=1.0)
            targets = [self.grad_accumulator.get_grad_buffer(n) if self.grad_accumulator is not None else p.grad for n, p in named]
            targets = [t for t in targets if t is not None]
            torch._foreach_mul_(targets, coef)
            return total
        return clip_grad_norm(mp_pg=ctx.mp_pg, named_parameters=named, grad_accumulator=self.grad_accumulator, max_norm=self.config.optimizer.clip_grad)

    def _move_optimizer_state_to_device(self):
        base = self.optimizer.get_base_optimizer()
        device = self.parallel_context.device
        for st in base.state.values():
            for k, v in st.items():
                if isinstance(v, torch.Tensor) and k != "step":
                    st[k] = v.to(device)

    def validation_step(self, dataloader) -> Iterable[Dict]:
        return self.pipeline_engine.validate_batch_iter(model=self.model, batch=(next(dataloader) for _ in range(self.limit_val_batches)), nb_microbatches=self.limit_val_batches)

    # ------------------------------------------------------------------ logging
    @property
    def logger_ranks(self):
        ctx = self.parallel_context
        return [int(ctx.get_global_rank(ep_rank=0, pp_rank=self.unwrapped_model.output_pp_rank, dp_rank=0, cp_rank=0, tp_rank=0))]

    def train_step_logs(self, outputs, loss_avg: Optional[torch.Tensor], z_loss_avg: Optional[torch.Tensor] = None) -> None:
        ctx = self.parallel_context
        dist.barrier(ctx.world_pg)
        self.iteration_timer.end()
        elapsed = torch.tensor([self.iteration_timer.elapsed], dtype=torch.float64, device=ctx.device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX, group=ctx.world_pg)  # the slowest rank defines the step time
        elapsed_ms = float(elapsed.item()) * 1000
        self.last_iteration_time_ms = elapsed_ms
        tokens_per_sec = self.global_batch_size * self.sequence_length / (elapsed_ms / 1000)
        model_tflops, hardware_tflops = self.unwrapped_model.get_flops_per_sec(iteration_time_in_sec=elapsed_ms / 1000, sequence_length=self.sequence_length, global_batch_size=self.global_batch_size)
        self.last_tokens_per_sec, self.last_model_tflops = tokens_per_sec, model_tflops
        if dist.get_rank(ctx.world_pg) in self.logger_ranks:
            assert loss_avg is not None
            lr = self.lr_scheduler.get_last_lr()[0]
            remaining = self.config.tokens.train_steps - self.iteration_step
            entries = [
                LogItem("consumed_tokens", self.metadata.consumed_tokens_total, "human_format"),
                LogItem("time_per_iteration_ms", elapsed_ms, "human_format"),
                LogItem("tokens_per_sec", tokens_per_sec, "human_format"),
                LogItem("tokens_per_sec_per_gpu", tokens_per_sec / ctx.world_pg.size(), "human_format"),
                LogItem("global_batch_size", self.global_batch_size, "human_format"),
                LogItem("lm_loss", loss_avg.item(), "human_format"),
            ]
            if z_loss_avg is not None:
                entries.append(LogItem("z_loss", z_loss_avg.item(), "human_format"))
            if self.grad_norm_unclipped is not None:
                entries.append(LogItem("grad_norm", self.grad_norm_unclipped.item(), "human_format"))
            entries += [
                LogItem("lr", lr, "human_format"),
                LogItem("model_tflops_per_gpu", model_tflops, "human_format"),
                LogItem("eta", str(datetime.timedelta(seconds=int(remaining * elapsed_ms / 1000))), None),
            ]
            if hardware_tflops != model_tflops:
                entries.append(LogItem("hardware_tflops_per_gpu", hardware_tflops, "human_format"))
            if nanotron_timer.is_enabled():
                for name, t in nanotron_timer.items():
                    if name != "iteration_time" and t.call_count:
                        entries.append(LogItem(f"timers/{name}", t.elapsed * 1000, ".2f"))
            if not hasattr(self, "loggerwriter"):
                self.loggerwriter = LoggerWriter(global_step=self.config.tokens.train_steps)
            self.loggerwriter.add_scalars_from_list(entries, self.iteration_step)
            # everything below goes to the metric sinks only (wandb, the JSONL file), not to the console line
            entries += self._diagnostic_log_items()
            if self._detailed_metrics is not None:
                entries += [LogItem(k, v, "human_format") for k, v in self._detailed_metrics.items()]
                self._detailed_metrics = None
            self._emit_metrics(entries)
        # (ranks other than the logger rank hold other shards and other layers: the training loop emits what they collected)
        if os.environ.get("NANOTRON_BENCHMARK", "0") == "1" and self.iteration_step == 4:
            log_throughput(self.config, ctx, model_tflops, hardware_tflops, tokens_per_sec, num_params=getattr(self, "num_params", {"total": 0, "local": 0}))
            log_rank("Throughput logging complete", logger=logger, level=logging.INFO, rank=0)
            if os.environ.get("NANOTRON_BENCHMARK_NO_EXIT", "0") != "1":
                raise SystemExit(0)

    def _is_metrics_rank(self) -> bool:
        """The ranks that report detailed metrics: the first data / context-parallel replica of every tensor-parallel rank and
        pipeline stage (each holds other shards and other layers; reference trainer.py:894-903)."""
        ctx = self.parallel_context
        return dist.get_rank(ctx.dp_pg) == 0 and dist.get_rank(ctx.cp_pg) == 0

    def _shard_suffix(self) -> str:
        """Names the model shard of this rank where several ranks report (detailed metrics under tp / pp > 1)."""
        ctx = self.parallel_context
        if self.metrics_logging.log_level == 0 or ctx.tp_pg.size() * ctx.pp_pg.size() == 1:
            return ""
        return f"pp{dist.get_rank(ctx.pp_pg)}_tp{dist.get_rank(ctx.tp_pg)}"

    def _diagnostic_log_items(self) -> List[LogItem]:
        """Optional entries: statistics of tensors that modules recorded with ``tbi_logger``, host memory (``DEBUG_CPU=1``),
        tokens drawn from every dataset folder (``DEBUG_DL=1``), device and disk memory."""
        items: List[LogItem] = []
        if hasattr(self.unwrapped_model, "get_tbi_logs"):
            for name, tensor in self.unwrapped_model.get_tbi_logs().items():
                t = tensor.float()
                if t.numel() == 0:
                    continue
                items += [LogItem(f"tbi_logs/{name}_{stat}", float(getattr(t, stat)()), "human_format") for stat in ("mean", "std", "max", "min")]
                if t.dim() >= 2:  # [heads, tokens]: one set per head
                    for h in range(t.shape[0]):
                        items += [LogItem(f"tbi_logs/{name}/head_{h}_{stat}", float(getattr(t[h], stat)()), "human_format") for stat in ("mean", "std", "max", "min")]
        if os.environ.get("DEBUG_CPU", "0") == "1":
            try:
                import psutil

                vm, proc = psutil.virtual_memory(), psutil.Process()
                items += [
                    LogItem("cpu_memory/total", vm.total, "human_format"), LogItem("cpu_memory/available", vm.available, "human_format"),
                    LogItem("cpu_memory/used_percent", vm.percent, ".1f"), LogItem("cpu_memory/process_rss", proc.memory_info().rss, "human_format"),
                ]
            except ImportError:
                pass
        if os.environ.get("DEBUG_DL", "0") == "1" and self.metadata.data_stages:
            stage = self.metadata.data_stages[self.metadata.last_stage_idx]
            items += [LogItem(f"dataloader/consumed_tokens/{folder}", tokens, "human_format") for folder, tokens in sorted(stage.consumed_tokens_per_dataset_folder.items())]
        if self.parallel_context.device.type == "cuda":
            items += [LogItem("cuda_memory_allocated", torch.cuda.memory_allocated(), "human_format"), LogItem("cuda_max_memory_reserved", torch.cuda.max_memory_reserved(), "human_format")]
        if self._detailed_metrics is not None:
            import shutil

            total, used, free = shutil.disk_usage(str(Path(self.config.checkpoints.checkpoints_path).anchor or "/"))
            items += [LogItem("hd_total_memory", total, "human_format"), LogItem("hd_used_memory", used, "human_format"), LogItem("hd_free_memory", free, "human_format")]
        return items

    def _emit_metrics(self, entries: List[LogItem]) -> None:
        record = {e.tag: e.scalar_value for e in entries}
        record["iteration_step"] = self.iteration_step
        suffix = self._shard_suffix()
        if suffix:
            ctx = self.parallel_context
            record.update(tp_rank=dist.get_rank(ctx.tp_pg), tp_group_size=ctx.tp_pg.size(), pp_rank=dist.get_rank(ctx.pp_pg))
        if getattr(self, "_wandb", None) is not None:
            self._wandb.log(record)
        if self._metrics_jsonl:
            with open(self._metrics_jsonl + (f".{suffix}" if suffix else ""), "a") as f:
                f.write(json.dumps(record, default=str) + "\n")

    # ------------------------------------------------------------------ model construction
    def init_model(self) -> NanotronModel:
        ctx = self.parallel_context
        if hasattr(self.model_config, "vocab_size"):
            self.model_config.vocab_size = _vocab_size_with_padding(self.model_config.vocab_size, pg_size=ctx.tp_pg.size(), make_vocab_size_divisible_by=self.config.model.make_vocab_size_divisible_by)
        if hasattr(self.model_config, "max_position_embeddings") and self.model_config.max_position_embeddings < self.config.tokens.sequence_length:
            log_rank(f"max_position_embeddings ({self.model_config.max_position_embeddings}) < sequence_length ({self.config.tokens.sequence_length}); raising it", logger=logger, level=logging.WARNING, rank=0)
            self.model_config.max_position_embeddings = self.config.tokens.sequence_length
        model = self._init_model_instance()
        model = self._load_model_checkpoint(model)
        return model

    def _init_model_instance(self) -> NanotronModel:
        model_cls = CONFIG_TO_MODEL_CLASS[self.model_config.__class__.__name__]
        return self._init_model(model_builder=lambda: model_cls(config=self.model_config, parallel_context=self.parallel_context, parallel_config=self.config.parallelism, random_states=self.random_states))

    def _init_model(self, model_builder: Callable[[], NanotronModel], target_pp_ranks: Optional[List[int]] = None) -> NanotronModel:
        config, ctx = self.config, self.parallel_context
        model = build_model(parallel_context=ctx, dtype=config.model.dtype, target_pp_ranks=target_pp_ranks, device=ctx.device, model_builder=model_builder)
        mark_tied_parameters(model=model, parallel_context=ctx, parallel_config=config.parallelism)
        # parameter counts
        num_local = sum(p.numel() for p in model.parameters())
        t = torch.tensor([float(num_local)], dtype=torch.float64, device=ctx.device)
        size_mb = torch.tensor([sum(p.numel() * p.element_size() for p in model.parameters()) / 1024**2], dtype=torch.float64, device=ctx.device)
        total = t.clone()
        dist.all_reduce(total, group=ctx.tp_pg)
        dist.all_reduce(total, group=ctx.pp_pg)
        self.num_params = {"total": int(total.item()), "local": num_local}
        log_rank(f"Total number of parameters: {human_format(self.num_params['total'])} ({size_mb.item():.2f}MiB local)", logger=logger, level=logging.INFO, rank=0)
        log_rank(f"Local number of parameters: {human_format(num_local)}", logger=logger, level=logging.INFO, group=ctx.dp_pg, rank=0)
        check_model_has_grad(model=model, parallel_context=ctx)
        sanity_check(root_module=model)
        return model

    def _load_model_checkpoint(self, model: NanotronModel) -> NanotronModel:
        ctx = self.parallel_context
        if self.init_checkpoint_path is not None:
            log_rank(f"Loading weights from {self.init_checkpoint_path}", logger=logger, level=logging.INFO, rank=0)
            self.param_shard_metadata = load_weights(model=model, parallel_context=ctx, root_folder=self.init_checkpoint_path)
            return model
        init = self.config.model.init_method
        if isinstance(init, ExistingCheckpointInit):
            log_rank(f"Loading weights from {init.path}", logger=logger, level=logging.INFO, rank=0)
            self.param_shard_metadata = load_weights(model=model, parallel_context=ctx, root_folder=init.path)
        elif isinstance(init, (RandomInit, SpectralMupInit)):
            model.init_model_randomly(config=self.config)
            # replicas must start identical: broadcast from dp rank 0 / the first rank of every tie group
            self._sync_initial_parameters(model)
        else:
            raise ValueError(f"Unsupported {init}")
        return model

    @torch.no_grad()
    def _sync_initial_parameters(self, model):
        ctx = self.parallel_context
        for name, p in sorted(model.named_parameters(), key=lambda x: x[0]):
            group = ctx.expert_dp_pg if self._param_is_expert(p) else ctx.dp_cp_pg
            if self._param_is_expert(p) and ctx.cp_pg.size() > 1:
                dist.broadcast(p.data, src=dist.get_global_rank(ctx.cp_pg, 0), group=ctx.cp_pg)
            if group.size() > 1:
                dist.broadcast(p.data, src=dist.get_global_rank(group, 0), group=group)
        for (_, ranks), p in sorted(get_tied_id_to_param(list(model.parameters()), root_module=model).items(), key=lambda x: x[0]):
            group = ctx.world_ranks_to_pg[tuple(sorted(ranks))]
            if group.size() > 1:
                dist.broadcast(p.data, src=sorted(ranks)[0], group=group)

    # ------------------------------------------------------------------ checkpoints
    def pre_save_checkpoint(self) -> Path:
        if self.s3_mover is not None:
            self.s3_mover.distributed_wait_for_completion(self.parallel_context.world_pg)
            if self.s3_mover.post_upload_callback_outputs is not None:
                slurm_job_id, slurm_log = self.s3_mover.post_upload_callback_outputs
                log_rank(f"launching eval job: job_id={slurm_job_id} log at {slurm_log} slurm_eval", logger=logger, level=logging.WARNING, rank=0)

    def post_save_checkpoint(self):
        if self.s3_mover is not None:
            self.s3_mover.start_uploading()

    def save_checkpoint(self) -> Path:
        self.pre_save_checkpoint()
        checkpoints_path = Path(self.config.checkpoints.checkpoints_path)
        checkpoint_path = checkpoints_path / f"{self.iteration_step}"
        ctx = self.parallel_context
        if self.config.checkpoints.checkpoints_path_is_shared_file_system:
            should_mkdir = dist.get_rank(ctx.world_pg) == 0
        else:
            should_mkdir = bool(int(os.environ.get("LOCAL_RANK", "0")) == 0)
        if should_mkdir:
            checkpoint_path.mkdir(parents=True, exist_ok=True)
        dist.barrier(ctx.world_pg)
        log_rank(f"Saving checkpoint at {checkpoint_path}", logger=logger, level=logging.WARNING, rank=0)
        self.config.general.step = self.metadata.last_train_step
        self.config.general.consumed_train_samples = self.metadata.consumed_train_samples
        save(
            model=self.unwrapped_model, optimizer=self.optimizer, lr_scheduler=self.lr_scheduler, should_save_model=True, should_save_optimizer=True,
            should_save_lr_scheduler=True, should_save_config=True, parallel_context=ctx, root_folder=checkpoint_path, training_metadata=self.metadata,
            config=self.config, sanity_checks=not self.config.general.ignore_sanity_checks,
        )
        save_random_states(random_states=self.random_states, parallel_context=ctx, root_folder=checkpoint_path)
        if dist.get_rank(ctx.world_pg) == 0:
            with open(checkpoints_path / LATEST_FILE_NAME, mode="w") as fo:
                fo.write(f"{self.iteration_step}")
            if hasattr(self.model_config, "to_json_file"):
                self.model_config.to_json_file(checkpoint_path / MODEL_CONFIG_FILE_NAME)
            else:
                with open(checkpoint_path / MODEL_CONFIG_FILE_NAME, mode="w") as fo:
                    d = asdict(self.model_config)
                    fo.write(json.dumps(d, default=str))
        dist.barrier(ctx.world_pg)
        self.post_save_checkpoint()
        return checkpoint_path


# ---------------------------------------------------------------------------- tying
def mark_tied_parameters(model: NanotronModel, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs] = None):
    """Tie embeddings with the lm head when the model asks for it, custom model ties, then every parameter that is
    replicated over tp (norm weights, router, biases of row linears)."""
    names = model.get_embeddings_lm_head_tied_names()
    if len(names) > 0:
        shared = [
            (
                target,
                (
                    int(parallel_context.get_global_rank(
                        ep_rank=0, pp_rank=get_pp_rank_of(target, module=model), dp_rank=dist.get_rank(parallel_context.dp_pg),
                        cp_rank=dist.get_rank(parallel_context.cp_pg), tp_rank=dist.get_rank(parallel_context.tp_pg),
                    )),
                ),
            )
            for target in names
        ]
        tie_parameters(root_module=model, ties=shared, parallel_context=parallel_context, reduce_op=dist.ReduceOp.SUM)
    model.tie_custom_params()
    mark_unsharded_params_as_tied_across_tp(model, parallel_context, parallel_config)
    mark_unsharded_params_as_tied_across_expert(model, parallel_context, parallel_config)
    create_pg_for_tied_weights(root_module=model, parallel_context=parallel_context)


def mark_unsharded_params_as_tied_across_tp(model: NanotronModel, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs]):
    tp_ranks = dist.get_global_ranks(parallel_context.tp_pg)
    for module_name, module in model.named_modules():
        for param_name, param in list(module.named_parameters(recurse=False)):
            name = f"{module_name}.{param_name}" if module_name else param_name
            if isinstance(param, NanotronParameter):
                if param.is_tied:
                    continue
                if param.is_sharded and not (param.get_sharded_info().is_expert_sharded(parallel_context) and parallel_context.tp_pg.size() > 1):
                    continue  # sharded over tp: distinct data per rank
                # (sharded over the expert axis only: the tp ranks hold copies of the same local experts, and under sequence
                # parallelism each copy sees a different token shard, so their gradients are summed like any replicated weight's)
            # ALL_REDUCE: activations are replicated so gradients are already identical (no reduction).
            # REDUCE_SCATTER: every tp rank saw different tokens, gradients must be summed.
            if parallel_config is None or parallel_config.tp_mode is TensorParallelLinearMode.ALL_REDUCE:
                reduce_op = None
            else:
                reduce_op = dist.ReduceOp.SUM
            if isinstance(module, TensorParallelRowLinear) and param_name == "bias":
                # the bias is added after the reduction on every rank with identical gradients
                reduce_op = None if (parallel_config is None or parallel_config.tp_mode is TensorParallelLinearMode.ALL_REDUCE) else dist.ReduceOp.SUM
            tie_parameters(root_module=model, ties=[(name, tp_ranks)], parallel_context=parallel_context, reduce_op=reduce_op)


def mark_unsharded_params_as_tied_across_expert(model: NanotronModel, parallel_context: ParallelContext, parallel_config: Optional[ParallelismArgs]):
    """Expert parallelism is laid over the data-parallel axis here, so parameters that are not expert-sharded are
    ordinary data-parallel replicas: they are kept in sync by the data-parallel gradient average and need no tie.
    Kept for API parity with the reference trainer."""
    return
