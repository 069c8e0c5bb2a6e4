"""Parallelism section of the config (schema parity: reference src/nanotron/config/parallelism_config.py:14-53; the field
names, their order and their defaults are the YAML contract)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from nanotron_b200.config.utils_config import cast_str_to_pipeline_engine
from nanotron_b200.parallel.pipeline_parallel.engine import AllForwardAllBackwardPipelineEngine, PipelineEngine
from nanotron_b200.parallel.tensor_parallel.enum import TensorParallelLinearMode

_SIZES = ("dp", "pp", "tp", "expert_parallel_size", "context_parallel_size")


@dataclass
class ParallelismArgs:
    dp: int  # data-parallel replicas
    pp: int  # pipeline stages
    tp: int  # tensor-parallel ranks (neighbouring GPUs)
    pp_engine: Optional[PipelineEngine] = None  # "afab" (default) or "1f1b"; a string is turned into the engine object
    tp_mode: Optional[TensorParallelLinearMode] = None  # ALL_REDUCE (default) or REDUCE_SCATTER = sequence parallelism
    tp_linear_async_communication: Optional[bool] = None  # collectives inside the GEMM kernels (default off)
    recompute_layer: bool = False  # recompute every decoder layer in the backward pass
    tp_recompute_allgather: bool = True  # keep only the split input of a column linear and gather it again for the backward
    expert_parallel_size: int = 1  # a sub-division of dp: experts are split over consecutive data-parallel ranks
    context_parallel_size: int = 1  # ranks that share one sequence
    # pipeline stages exchange tensor headers only during the first micro-batch and replay the learnt shapes afterwards
    # (every micro-batch of a data stage has the same geometry); False sends a header with every activation
    pp_static_shapes: bool = True

    def __post_init__(self):
        for name in _SIZES:
            size = getattr(self, name)
            if not isinstance(size, int) or size < 1:
                raise ValueError(f"parallelism.{name} must be a positive integer, got {size!r}")
        if self.dp % self.expert_parallel_size != 0:
            raise ValueError(f"parallelism.expert_parallel_size ({self.expert_parallel_size}) must divide parallelism.dp ({self.dp}): expert ranks are a sub-division of the data-parallel ranks")
        engine = self.pp_engine if self.pp_engine is not None else AllForwardAllBackwardPipelineEngine()
        self.pp_engine = cast_str_to_pipeline_engine(engine) if isinstance(engine, str) else engine
        mode = self.tp_mode if self.tp_mode is not None else TensorParallelLinearMode.ALL_REDUCE
        self.tp_mode = TensorParallelLinearMode[mode.upper()] if isinstance(mode, str) else mode
        self.tp_linear_async_communication = bool(self.tp_linear_async_communication)

    @property
    def world_size(self) -> int:
        """Processes this layout needs (expert parallelism re-uses the data-parallel ranks)."""
        return self.dp * self.pp * self.tp * self.context_parallel_size

    def describe(self) -> str:
        """``dp2 x tp4 (sequence parallel) x pp2 (1f1b)``: the layout in one line, for logs."""
        parts = [f"dp{self.dp}"]
        if self.expert_parallel_size > 1:
            parts[-1] += f" (ep{self.expert_parallel_size})"
        if self.context_parallel_size > 1:
            parts.append(f"cp{self.context_parallel_size}")
        if self.tp > 1:
            parts.append(f"tp{self.tp}" + (" (sequence parallel)" if self.tp_mode == TensorParallelLinearMode.REDUCE_SCATTER else ""))
        if self.pp > 1:
            parts.append(f"pp{self.pp} ({type(self.pp_engine).__name__})")
        return " x ".join(parts)
