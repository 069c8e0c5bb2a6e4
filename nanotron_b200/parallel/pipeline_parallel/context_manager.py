from contextlib import contextmanager

from torch import nn as torch_nn

from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock
from nanotron_b200.parallel.pipeline_parallel.state import PipelineBatchState


@contextmanager
def attach_pipeline_state_to_model(model: torch_nn.Module, pipeline_state: PipelineBatchState):
    """Give every PipelineBlock of ``model`` access to ``pipeline_state`` for the duration of the block."""
    blocks = [m for m in model.modules() if isinstance(m, PipelineBlock)]
    old = [b.pipeline_state for b in blocks]
    for b in blocks:
        b.set_pipeline_state(pipeline_state)
    try:
        yield
    finally:
        for b, o in zip(blocks, old):
            b.set_pipeline_state(o)
