"""``PipelineBlock``: a module that exists on exactly one pipeline rank (parity: reference
src/nanotron/parallel/pipeline_parallel/block.py:16-185).

Every rank declares every block; ``build_and_set_rank`` instantiates the wrapped module only on the owner.
Calling a block on a non-owner rank forwards real tensors to the owner and returns ``TensorPointer``s; calling it
on the owner receives the inputs that are pointers, runs the module and returns real tensors.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Set, Tuple, Union

import torch
from torch import nn

from nanotron_b200 import distributed as dist
from nanotron_b200.parallel.pipeline_parallel.functional import (
    recv_from_pipeline_state_buffer,
    send_to_pipeline_state_buffer,
)
from nanotron_b200.parallel.pipeline_parallel.p2p import P2P, BatchTensorSendRecvState
from nanotron_b200.parallel.pipeline_parallel.state import PipelineBatchState, PipelineTrainBatchState
from nanotron_b200.parallel.pipeline_parallel.tensor_pointer import TensorPointer


class PipelineBlock(nn.Module):
    def __init__(
        self,
        p2p: P2P,
        module_builder: Callable[..., nn.Module],
        module_kwargs: Dict[str, Any],
        module_input_keys: Set[str],
        module_output_keys: Set[str],
    ):
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

    def forward(self, **kwargs):
        assert self.module_input_keys == set(kwargs.keys()), f"Expected {self.module_input_keys}, got {set(kwargs.keys())}"
        me = dist.get_rank(self.p2p.pg)
        sorted_kwargs = sorted(kwargs.items(), key=get_sort_key(me))
        if me != self.rank:
            # non-owner: ship the tensors I hold to the owner, answer with pointers
            batch_send_recv = BatchTensorSendRecvState(self.p2p)
            for name, tensor in sorted_kwargs:
                if isinstance(tensor, TensorPointer):
                    continue
                if isinstance(tensor, torch.Tensor):
                    if self.pipeline_state is not None:
                        send_to_pipeline_state_buffer(tensor, to_rank=self.rank, p2p=self.p2p, pipeline_state=self.pipeline_state)
                    else:
                        assert not tensor.requires_grad, "Sending a tensor that requires grad needs a pipeline state"
                        batch_send_recv.add_send(tensor=tensor, to_rank=self.rank)
                # non-tensor values are known on every rank: nothing to send
            batch_send_recv.flush()
            return {k: TensorPointer(group_rank=self.rank) for k in self.module_output_keys}
        # owner
        new_kwargs: Dict[str, Any] = {}
        name_to_recv_id = {}
        batch_send_recv = BatchTensorSendRecvState(self.p2p)
        for name, tensor in sorted_kwargs:
            if isinstance(tensor, TensorPointer):
                if self.pipeline_state is not None:
                    new_kwargs[name] = recv_from_pipeline_state_buffer(from_rank=tensor.group_rank, p2p=self.p2p, pipeline_state=self.pipeline_state)
                    continue
                name_to_recv_id[name] = batch_send_recv.add_recv(from_rank=tensor.group_rank)
                continue
            new_kwargs[name] = tensor
        received = batch_send_recv.flush()
        for name, idx in name_to_recv_id.items():
            t = received[idx]
            assert not t.requires_grad, "Receiving a tensor that requires grad needs a pipeline state"
            new_kwargs[name] = t
        output = self.pp_block(**new_kwargs)
        if isinstance(output, torch.Tensor):
            assert len(self.module_output_keys) == 1
            output = {next(iter(self.module_output_keys)): output}
        assert isinstance(output, dict), "Modules within a PipelineBlock have to return a Dict[str, torch.Tensor]"
        assert self.module_output_keys == set(output.keys()), f"Expected {self.module_output_keys}, got {set(output.keys())}"
        return output


def get_min_max_rank(module: nn.Module) -> Tuple[int, int]:
    ranks = [m.rank for m in module.modules() if isinstance(m, PipelineBlock)]
    return min(ranks), max(ranks)


def get_sort_key(current_rank: int):
    """Order kwargs so sends/recvs between two ranks are issued in the same order on both sides: tensors held here
    sort by (this rank, name), pointers by (their rank, name)."""

    def sort_key(elt: Tuple[str, Union[torch.Tensor, TensorPointer]]):
        name, tensor = elt
        rank = tensor.group_rank if isinstance(tensor, TensorPointer) else current_rank
        return rank, name

    return sort_key
