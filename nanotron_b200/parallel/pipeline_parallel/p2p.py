"""Point-to-point tensor exchange between pipeline stages (NCCL or gloo send/recv).

Wire format per tensor: ONE fixed-size int64 header followed by the payload.
    header = [ndim, dtype_id, requires_grad, numel, d0, d1, ... d7]      (12 x int64)
The payload is always sent contiguous, so no stride/storage description is needed; complex tensors travel as
their real view.  This replaces the reference's two variable-length metadata messages per tensor
(reference src/nanotron/parallel/pipeline_parallel/p2p.py:80-98,289-356) and keeps its API:
``isend_tensors / irecv_tensors / send_tensors / recv_tensors`` and ``BatchTensorSendRecvState``.

When both sides declare static shapes with :meth:`P2P.expect_static`, headers are exchanged only the first time
a (peer, direction, tag) triple is used and replayed from a cache afterwards: steady-state pipeline traffic is
then one message per tensor.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.logging import get_logger

logger = get_logger(__name__)

MAX_NDIM = 8
HEADER_LEN = 4 + MAX_NDIM
DTYPE_TO_ID = {
    torch.float32: 0,
    torch.float64: 1,
    torch.complex64: 2,
    torch.complex128: 3,
    torch.float16: 4,
    torch.bfloat16: 5,
    torch.uint8: 6,
    torch.int8: 7,
    torch.int16: 8,
    torch.int32: 9,
    torch.int64: 10,
    torch.bool: 11,
    torch.float8_e4m3fn: 12,
    torch.float8_e5m2: 13,
}
ID_TO_DTYPE = {v: k for k, v in DTYPE_TO_ID.items()}


@dataclasses.dataclass
class P2PTensorMetaData:
    shape: Tuple[int, ...]
    dtype: torch.dtype
    requires_grad: bool

    def to_header(self, device) -> torch.Tensor:
        assert len(self.shape) <= MAX_NDIM, f"tensors with more than {MAX_NDIM} dims are not supported over p2p"
        numel = 1
        for s in self.shape:
            numel *= s
        vals = [len(self.shape), DTYPE_TO_ID[self.dtype], int(self.requires_grad), numel, *self.shape]
        vals += [0] * (HEADER_LEN - len(vals))
        return torch.tensor(vals, dtype=torch.long, device=device)

    @staticmethod
    def from_header(header: torch.Tensor) -> "P2PTensorMetaData":
        vals = header.tolist()
        ndim = vals[0]
        return P2PTensorMetaData(shape=tuple(vals[4 : 4 + ndim]), dtype=ID_TO_DTYPE[vals[1]], requires_grad=bool(vals[2]))

    def create_empty_storage(self, device) -> torch.Tensor:
        dtype = self.dtype
        return torch.empty(self.shape, dtype=dtype, device=device, requires_grad=False)

    @staticmethod
    def from_tensor(t: torch.Tensor) -> "P2PTensorMetaData":
        return P2PTensorMetaData(shape=tuple(t.shape), dtype=t.dtype, requires_grad=t.requires_grad)


def _wire_view(t: torch.Tensor) -> torch.Tensor:
    if t.is_complex():
        return torch.view_as_real(t)
    if t.dtype == torch.bool:
        return t.view(torch.uint8)
    return t


class P2P:
    def __init__(self, pg: dist.ProcessGroup, device: torch.device):
        self.pg = pg
        self.device = device
        self._static = False
        self._send_cache: Dict[Tuple[int, int], P2PTensorMetaData] = {}
        self._recv_cache: Dict[Tuple[int, int], P2PTensorMetaData] = {}

    def expect_static(self, enabled: bool = True):
        """Both peers promise that the i-th tensor exchanged under a given tag keeps its shape/dtype; headers are
        then sent once.  Must be set identically on every rank of the group."""
        self._static = enabled
        if not enabled:
            self._send_cache.clear()
            self._recv_cache.clear()

    # ------------------------------------------------------------------ single tensor
    def _isend(self, tensor: torch.Tensor, to_rank: int, tag: int) -> List[dist.Work]:
        meta = P2PTensorMetaData.from_tensor(tensor)
        dst = dist.get_global_rank(self.pg, to_rank)
        futures = []
        key = (to_rank, tag)
        if not (self._static and self._send_cache.get(key) == meta):
            if self._static and key in self._send_cache:
                raise RuntimeError(f"p2p static-shape contract broken for peer {to_rank} tag {tag}: {self._send_cache[key]} -> {meta}")
            dist.send(meta.to_header(self.device), dst=dst, group=self.pg, tag=tag)
            if self._static:
                self._send_cache[key] = meta
        payload = _wire_view(tensor.detach()).contiguous()
        futures.append(dist.isend(payload, dst=dst, group=self.pg, tag=tag))
        self._keepalive = getattr(self, "_keepalive", [])
        self._keepalive.append(payload)
        if len(self._keepalive) > 64:
            self._keepalive = self._keepalive[-32:]
        return futures

    def _irecv(self, from_rank: int, tag: int) -> Tuple[torch.Tensor, List[dist.Work]]:
        src = dist.get_global_rank(self.pg, from_rank)
        key = (from_rank, tag)
        if self._static and key in self._recv_cache:
            meta = self._recv_cache[key]
        else:
            header = torch.empty(HEADER_LEN, dtype=torch.long, device=self.device)
            dist.recv(header, src=src, group=self.pg, tag=tag)
            meta = P2PTensorMetaData.from_header(header)
            if self._static:
                self._recv_cache[key] = meta
        buf = meta.create_empty_storage(self.device)
        work = dist.irecv(_wire_view(buf), src=src, group=self.pg, tag=tag)
        if meta.requires_grad:
            buf.requires_grad_(True)
        return buf, [work]

    # ------------------------------------------------------------------ public API
    def isend_tensors(self, tensors: List[torch.Tensor], to_rank: int, tag: int = 0) -> List[dist.Work]:
        futures = []
        for t in tensors:
            futures.extend(self._isend(t, to_rank, tag))
        return futures

    def irecv_tensors(self, num_tensors: int, from_rank: int, tag: int = 0) -> Tuple[List[torch.Tensor], List[dist.Work]]:
        tensors, futures = [], []
        for _ in range(num_tensors):
            t, f = self._irecv(from_rank, tag)
            tensors.append(t)
            futures.extend(f)
        return tensors, futures

    def send_tensors(self, tensors: List[torch.Tensor], to_rank: int, tag: int = 0):
        for f in self.isend_tensors(tensors, to_rank, tag):
            f.wait()

    def recv_tensors(self, num_tensors: int, from_rank: int, tag: int = 0) -> List[torch.Tensor]:
        tensors, futures = self.irecv_tensors(num_tensors, from_rank, tag)
        for f in futures:
            f.wait()
        return tensors


class BatchTensorSendRecvState:
    """Queue sends and receives, then run them together (``flush``): all headers as one ``batch_isend_irecv``,
    then all payloads as another, so opposite-direction transfers cannot deadlock."""

    def __init__(self, p2p: P2P):
        self.p2p = p2p
        self._reset()

    def _reset(self):
        self.send_queue: List[Tuple[torch.Tensor, int]] = []
        self.recv_queue: List[int] = []

    def add_send(self, tensor: torch.Tensor, to_rank: int, tag: int = 0):
        self.send_queue.append((tensor, to_rank))

    def add_recv(self, from_rank: int, tag: int = 0) -> int:
        self.recv_queue.append(from_rank)
        return len(self.recv_queue) - 1

    def flush(self) -> List[torch.Tensor]:
        p2p = self.p2p
        if not self.send_queue and not self.recv_queue:
            return []
        # phase 1: every header in one batched exchange (deadlock-free whatever the peer pattern)
        send_headers = [P2PTensorMetaData.from_tensor(t).to_header(p2p.device) for t, _ in self.send_queue]
        recv_headers = [torch.empty(HEADER_LEN, dtype=torch.long, device=p2p.device) for _ in self.recv_queue]
        hops = [dist.P2POp(dist.isend, h, dist.get_global_rank(p2p.pg, to), group=p2p.pg) for h, (_, to) in zip(send_headers, self.send_queue)]
        hops += [dist.P2POp(dist.irecv, h, dist.get_global_rank(p2p.pg, frm), group=p2p.pg) for h, frm in zip(recv_headers, self.recv_queue)]
        for w in dist.batch_isend_irecv(hops):
            w.wait()
        recv_meta = [P2PTensorMetaData.from_header(h) for h in recv_headers]
        # phase 2: payloads
        ops, bufs, keep = [], [], []
        for (t, to) in self.send_queue:
            payload = _wire_view(t.detach()).contiguous()
            keep.append(payload)
            ops.append(dist.P2POp(dist.isend, payload, dist.get_global_rank(p2p.pg, to), group=p2p.pg))
        for meta, frm in zip(recv_meta, self.recv_queue):
            buf = meta.create_empty_storage(p2p.device)
            bufs.append((buf, meta))
            ops.append(dist.P2POp(dist.irecv, _wire_view(buf), dist.get_global_rank(p2p.pg, frm), group=p2p.pg))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        out = []
        for buf, meta in bufs:
            if meta.requires_grad:
                buf.requires_grad_(True)
            out.append(buf)
        self._reset()
        return out
