"""Symmetric (peer-mapped) device memory for a node-local process group.

``SymmetricAllocator(group)`` hands out tensors whose storage every rank of ``group`` can address directly over
NVLink: after ``rendezvous`` each rank knows the device pointer of every peer's copy.  Kernels in
``nanotron_b200/ops/csrc/comm.cu`` take those pointer tables and do the collective themselves (peer loads / stores)
fused with their compute.  The mapping itself (CUDA virtual-memory allocation + handle exchange) is delegated to
``torch.distributed._symmetric_memory``; this module owns the flag words, the epoch-based barrier and the bounded-wait
error reporting.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

import nanotron_b200.distributed as dist

DEFAULT_WAIT_LIMIT_NS = 20_000_000_000  # a rank may be several seconds late (first-step lazy initialisation)


class CommTimeoutError(RuntimeError):
    """A device-side wait on a peer ran out; the context is still usable."""


def is_available(group) -> bool:
    if not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except ImportError:
        return False
    from nanotron_b200.ops import native

    if not native.available():
        return False
    return group.size() <= native.lib().ntb_comm_max_ranks()


class SymmetricTensor:
    """A local tensor plus the table of every rank's base pointer for the same allocation."""

    def __init__(self, tensor: torch.Tensor, handle, group):
        self.tensor = tensor
        self.handle = handle
        self.group = group
        self.world = group.size()
        self.rank = dist.get_rank(group)
        base = [int(p) for p in handle.buffer_ptrs]
        # `tensor` may start at an offset inside the symmetric allocation
        off = tensor.data_ptr() - base[self.rank]
        self.ptrs = (ctypes.c_uint64 * self.world)(*[b + off for b in base])

    def peer_table(self):
        return self.ptrs


class SymmetricAllocator:
    def __init__(self, group):
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group = group
        self.world = group.size()
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._registry: Dict[int, SymmetricTensor] = {}
        flags = self.zeros(max(self.world, 32), torch.int32)
        self.flags = flags
        self.epoch = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.wait_limit_ns = DEFAULT_WAIT_LIMIT_NS
        dist.barrier(group)  # flag words are zero everywhere before the first device barrier

    def zeros(self, numel: int, dtype: torch.dtype) -> SymmetricTensor:
        """Collective over the group: every rank must call it with the same arguments in the same order."""
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        handle = self._symm.rendezvous(t, self.group)
        st = SymmetricTensor(t, handle, self.group)
        self._registry[t.data_ptr()] = st
        return st

    def lookup(self, tensor: torch.Tensor) -> Optional[SymmetricTensor]:
        """Pointer table for a tensor that is (a view at the start of) one of this allocator's allocations."""
        return self._registry.get(tensor.data_ptr())

    def barrier(self):
        """Device-side barrier on the current stream (no host synchronisation)."""
        from nanotron_b200.ops import native

        self.epoch += 1
        with torch.cuda.device(self.device):
            rc = native.lib().ntb_symm_barrier(self.flags.ptrs, self.rank, self.world, self.epoch, self.wait_limit_ns, self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "symm_barrier")

    def check(self):
        """Host-side check of the status word (synchronises the stream)."""
        v = int(self.status.item())
        if v != 0:
            self.status.zero_()
            raise CommTimeoutError(f"a peer did not reach the barrier within {self.wait_limit_ns / 1e9:.1f} s (status {v})")
