"""Parallelism section of the config (parity: reference src/nanotron/config/parallelism_config.py:14-53)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from nanotron_b200.config.utils_config import cast_str_to_pipeline_engine
from nanotron_b200.parallel.pipeline_parallel.engine import AllForwardAllBackwardPipelineEngine, PipelineEngine
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode


@dataclass
class ParallelismArgs:
    """
    dp / pp / tp: group sizes.  pp_engine: "1f1b" or "afab".  tp_mode: "all_reduce" or "reduce_scatter"
    (the latter is sequence parallelism).  tp_linear_async_communication: overlap the TP collectives with the
    GEMMs (fused kernels on GPU).  recompute_layer: recompute each decoder layer in backward.
    expert_parallel_size must divide dp (experts are sharded over consecutive dp ranks).
    zero_fused_comm: use the in-kernel reduce-scatter + AdamW + all-gather path over peer memory for ZeRO-1.
    """

    dp: int
    pp: int
    tp: int
    pp_engine: Optional[PipelineEngine] = None
    tp_mode: Optional[TensorParallelLinearMode] = None
    tp_linear_async_communication: Optional[bool] = None
    recompute_layer: bool = False
    tp_recompute_allgather: bool = True
    expert_parallel_size: int = 1
    context_parallel_size: int = 1
    # pipeline stages exchange tensor headers only during the first micro-batch and replay the learnt shapes afterwards
    # (every micro-batch of a data stage has the same geometry); False sends a header with every activation
    pp_static_shapes: bool = True

    def __post_init__(self):
        if self.pp_engine is None:
            self.pp_engine = AllForwardAllBackwardPipelineEngine()
        if self.tp_mode is None:
            self.tp_mode = TensorParallelLinearMode.ALL_REDUCE
        if self.tp_linear_async_communication is None:
            self.tp_linear_async_communication = False
        if isinstance(self.pp_engine, str):
            self.pp_engine = cast_str_to_pipeline_engine(self.pp_engine)
        if isinstance(self.tp_mode, str):
            self.tp_mode = TensorParallelLinearMode[self.tp_mode.upper()]
