"""Pipeline helpers (parity: reference src/nanotron/parallel/pipeline_parallel/utils.py)."""
from torch import nn
from torch.nn.parallel import DistributedDataParallel


def get_input_output_pp_ranks(model):
    """pp ranks of the first and last PipelineBlock of ``model``."""
    from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

    if isinstance(model, DistributedDataParallel):
        model = model.module
    blocks = [m for m in model.modules() if isinstance(m, PipelineBlock)]
    return blocks[0].rank, blocks[-1].rank


def get_pp_rank_of(target: str, module: nn.Module) -> int:
    """pp rank holding the parameter/module named ``target`` (walks up to the enclosing PipelineBlock)."""
    from nanotron_b200.parallel.pipeline_parallel.block import PipelineBlock

    if isinstance(module, PipelineBlock):
        return module.rank
    path = target.split(".")
    current = module
    for name in path:
        if not hasattr(current, name):
            break
        current = getattr(current, name)
        if isinstance(current, PipelineBlock):
            return current.rank
    raise ValueError(f'Module with name "{target}" can\'t be found inside a PipelineBlock.')
