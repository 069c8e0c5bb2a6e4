"""``PipelineBlock``: a module that lives on exactly one pipeline rank (API parity: reference
src/nanotron/parallel/pipeline_parallel/block.py:16-185).

Every rank declares every block of the model; ``build_and_set_rank`` instantiates the wrapped module on its owner only.
A call on the owner turns ``TensorPointer`` arguments into real tensors (received from the rank the pointer names), runs the
module and returns real tensors; a call anywhere else ships the real tensors this rank holds to the owner and returns
pointers to the owner.  With a pipeline state attached the traffic goes through it (so a schedule can account for
gradients); without one, tensors that need no gradient are exchanged on the spot in one batched send/recv.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Set, Tuple, Union

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200.parallel.pipeline_parallel.functional import recv_from_pipeline_state_buffer, send_to_pipeline_state_buffer
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P, BatchTensorSendRecvState
from nanotron_b200.parallel.pipeline_parallel.state import PipelineBatchState
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer


class PipelineBlock(nn.Module):
    def __init__(self, p2p: P2P, module_builder: Callable[..., nn.Module], module_kwargs: Dict[str, Any], module_input_keys: Set[str], module_output_keys: Set[str]):
        super().__init__()
        self.p2p = p2p
        self.module_builder = module_builder
        self.module_kwargs = module_kwargs
        self.module_input_keys = set(module_input_keys)
        self.module_output_keys = set(module_output_keys)
        self.pipeline_state: Optional[PipelineBatchState] = None
        self.rank: Optional[int] = None

    def build_and_set_rank(self, pp_rank: int):
        assert pp_rank < self.p2p.pg.size()
        self.rank = pp_rank
        if pp_rank == dist.get_rank(self.p2p.pg):
            self.pp_block = self.module_builder(**self.module_kwargs)

    def extra_repr(self) -> str:
        return f"pp_rank={self.rank}" if self.rank is not None else ""

    def set_pipeline_state(self, pipeline_state: Optional[PipelineBatchState]):
        self.pipeline_state = pipeline_state

    # ------------------------------------------------------------------ the two roles
    def _forward_to_owner(self, ordered: List[Tuple[str, Any]]) -> Dict[str, TensorPointer]:
        immediate = BatchTensorSendRecvState(self.p2p)
        for _, value in ordered:
            if not isinstance(value, torch.Tensor):
                continue  # pointers are someone else's to send; plain python values are known everywhere
            if self.pipeline_state is not None:
                send_to_pipeline_state_buffer(value, to_rank=self.rank, p2p=self.p2p, pipeline_state=self.pipeline_state)
            else:
                assert not value.requires_grad, "Sending a tensor that requires grad needs a pipeline state"
                immediate.add_send(tensor=value, to_rank=self.rank)
        immediate.flush()
        return {key: TensorPointer(group_rank=self.rank) for key in self.module_output_keys}

    def _run_as_owner(self, ordered: List[Tuple[str, Any]]) -> Dict[str, torch.Tensor]:
        resolved: Dict[str, Any] = {}
        immediate = BatchTensorSendRecvState(self.p2p)
        awaiting: Dict[str, int] = {}
        for name, value in ordered:
            if not isinstance(value, TensorPointer):
                resolved[name] = value
            elif self.pipeline_state is not None:
                resolved[name] = recv_from_pipeline_state_buffer(from_rank=value.group_rank, p2p=self.p2p, pipeline_state=self.pipeline_state)
            else:
                awaiting[name] = immediate.add_recv(from_rank=value.group_rank)
        arrived = immediate.flush()
        for name, idx in awaiting.items():
            assert not arrived[idx].requires_grad, "Receiving a tensor that requires grad needs a pipeline state"
            resolved[name] = arrived[idx]
        output = self.pp_block(**resolved)
        if isinstance(output, torch.Tensor):
            assert len(self.module_output_keys) == 1
            output = {next(iter(self.module_output_keys)): output}
        assert isinstance(output, dict), "Modules within a PipelineBlock have to return a Dict[str, torch.Tensor]"
        assert self.module_output_keys == set(output.keys()), f"Expected {self.module_output_keys}, got {set(output.keys())}"
        return output

    def forward(self, **kwargs):
        assert self.module_input_keys == set(kwargs.keys()), f"Expected {self.module_input_keys}, got {set(kwargs.keys())}"
        me = dist.get_rank(self.p2p.pg)
        ordered = sorted(kwargs.items(), key=get_sort_key(me))
        return self._run_as_owner(ordered) if me == self.rank else self._forward_to_owner(ordered)


def get_min_max_rank(module: nn.Module) -> Tuple[int, int]:
    ranks = [m.rank for m in module.modules() if isinstance(m, PipelineBlock)]
    return min(ranks), max(ranks)


def get_sort_key(current_rank: int):
    """Both ends of a boundary must walk the arguments in the same order: a tensor held here sorts under this rank, a pointer
    under the rank it names, ties broken by argument name."""

    def sort_key(item: Tuple[str, Union[torch.Tensor, TensorPointer]]):
        name, value = item
        return (value.group_rank if isinstance(value, TensorPointer) else current_rank), name

    return sort_key
