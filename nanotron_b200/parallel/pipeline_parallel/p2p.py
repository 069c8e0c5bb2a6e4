"""Point-to-point tensor exchange between pipeline stages (NCCL or gloo send/recv).

Two lanes per stage boundary
    Activations travel stage s -> s+1 on the *forward lane*, gradients s+1 -> s on the *backward lane*; each lane is a
    process group of its own (``register_lanes``; ``ParallelContext`` creates them when pp > 1).  A lane between two
    ranks is therefore one-directional during training: the i-th send on one side always meets the i-th receive on the
    other, whatever the schedule interleaves in between, so no ordering protocol between the two directions is needed
    and a gradient can leave as soon as it exists.  (The reference multiplexes both directions over one group and
    relies on every rank draining its queues in one fixed order: src/nanotron/parallel/pipeline_parallel/state.py:124-172.)

Wire format
    ONE fixed-size int64 header, then the payload, always contiguous:
        header = [ndim, dtype_id, requires_grad, numel, d0 ... d7]            (12 x int64)
    (reference: two variable-length metadata messages per tensor, p2p.py:80-98,289-356).  Two kinds of transfer send
    no header at all: gradients (shape and dtype are those of the activation they belong to: ``recv_like`` /
    ``send_raw``), and, once ``expect_static`` is on, activations whose per-micro-batch sequence of shapes was learnt
    during the first micro-batch (``begin_round`` marks the micro-batch boundaries).  Steady-state pipeline traffic is
    then one message per tensor and involves no host synchronisation.

Completion
    Sends never block the computing stream: the handle and the payload are parked in ``_inflight`` and retired by
    ``drain`` (end of a batch) or when the list grows.  Receives return a ``Ticket``; ``Ticket.wait`` makes the current
    stream wait for the data at first use.

The reference's API names are kept: ``isend_tensors / irecv_tensors / send_tensors / recv_tensors`` and
``BatchTensorSendRecvState`` (always with headers, forward lane).
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Deque, Dict, List, Optional, Tuple

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

FWD, BWD = "fwd", "bwd"
_LANES: Dict[int, Dict[str, dist.ProcessGroup]] = {}


def register_lanes(pg: dist.ProcessGroup, fwd_pg: dist.ProcessGroup, bwd_pg: dist.ProcessGroup) -> None:
    """Declare the two one-directional process groups (same ranks as ``pg``) that carry ``pg``'s pipeline traffic."""
    _LANES[id(pg)] = {FWD: fwd_pg, BWD: bwd_pg}


def lane_group(pg: dist.ProcessGroup, lane: str) -> dist.ProcessGroup:
    """Group to use for ``lane``; a group without registered lanes carries both directions itself."""
    lanes = _LANES.get(id(pg))
    return pg if lanes is None else lanes[lane]


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
        return torch.empty(self.shape, dtype=self.dtype, device=device, requires_grad=False)

    @staticmethod
    def from_tensor(t: torch.Tensor) -> "P2PTensorMetaData":
        return P2PTensorMetaData(shape=tuple(t.shape), dtype=t.dtype, requires_grad=t.requires_grad)


def _wire_view(t: torch.Tensor) -> torch.Tensor:
    if t.is_complex():
        return torch.view_as_real(t)
    if t.dtype == torch.bool:
        return t.view(torch.uint8)
    return t


class Ticket:
    """A receive that was posted; ``wait`` returns the tensor once the current stream may read it."""

    __slots__ = ("tensor", "works", "requires_grad")

    def __init__(self, tensor: torch.Tensor, works: List[dist.Work], requires_grad: bool):
        self.tensor, self.works, self.requires_grad = tensor, works, requires_grad

    def wait(self) -> torch.Tensor:
        for w in self.works:
            w.wait()
        self.works = []
        if self.requires_grad and not self.tensor.requires_grad:
            self.tensor.requires_grad_(True)
        return self.tensor


class _Pattern:
    """Shapes of the tensors exchanged with one peer in one direction on one lane during a micro-batch, learnt while the first
    micro-batch runs and replayed afterwards."""

    __slots__ = ("metas", "pos", "frozen")

    def __init__(self):
        self.metas: List[P2PTensorMetaData] = []
        self.pos = 0
        self.frozen = False


class P2P:
    def __init__(self, pg: dist.ProcessGroup, device: torch.device):
        self.pg = pg
        self.device = device
        self._static = False
        self._patterns: Dict[Tuple[str, int, str], _Pattern] = {}
        self._tag_cache: Dict[Tuple[str, int, int], P2PTensorMetaData] = {}
        self._inflight: Deque[Tuple[dist.Work, torch.Tensor]] = collections.deque()

    # ------------------------------------------------------------------ static shapes
    def expect_static(self, enabled: bool = True):
        """Both peers promise that every micro-batch exchanges the same sequence of shapes / dtypes (and, for the tagged
        reference-style calls, that a tag keeps its shape): headers are then sent once.  Must be set identically on
        every rank of the group, between batches."""
        self._static = enabled
        self.reset_static()

    def reset_static(self):
        """Forget the learnt shapes (call on every rank at a batch boundary when the batch geometry changes)."""
        self._patterns.clear()
        self._tag_cache.clear()

    def begin_round(self):
        """A new micro-batch starts: learnt sequences replay from their first element, and what the finished micro-batch
        exchanged becomes the contract for the following ones."""
        for p in self._patterns.values():
            if p.metas:
                p.frozen = True
            p.pos = 0

    def _pattern(self, direction: str, peer: int, lane: str) -> Optional[_Pattern]:
        if not self._static:
            return None
        key = (direction, peer, lane)
        p = self._patterns.get(key)
        if p is None:
            p = self._patterns[key] = _Pattern()
        return p

    # ------------------------------------------------------------------ lane transfers (pipeline engines)
    def _park(self, work: dist.Work, payload: torch.Tensor):
        self._inflight.append((work, payload))
        while len(self._inflight) > 64:
            w, _ = self._inflight.popleft()
            w.wait()  # by now long complete: orders nothing new, only releases the payload

    def drain(self):
        """Retire every send posted so far (their receives have been posted by the time a batch ends)."""
        while self._inflight:
            w, _ = self._inflight.popleft()
            w.wait()

    def send(self, tensor: torch.Tensor, to_rank: int, lane: str = FWD) -> None:
        """Asynchronous send with a header, or without one when the learnt pattern covers it."""
        group = lane_group(self.pg, lane)
        dst = dist.get_global_rank(self.pg, to_rank)
        meta = P2PTensorMetaData.from_tensor(tensor)
        pat = self._pattern("send", to_rank, lane)
        need_header = True
        if pat is not None:
            if pat.frozen:
                if pat.pos >= len(pat.metas) or pat.metas[pat.pos] != meta:
                    expected = pat.metas[pat.pos] if pat.pos < len(pat.metas) else "nothing"
                    raise RuntimeError(f"p2p static-shape contract broken towards pipeline rank {to_rank} ({lane} lane, tensor #{pat.pos} of the micro-batch): expected {expected}, got {meta}; call reset_static() on every rank when the batch geometry changes")
                need_header = False
            else:
                pat.metas.append(meta)
            pat.pos += 1
        if need_header:
            header = meta.to_header(self.device)
            self._park(dist.isend(header, dst=dst, group=group), header)
        self.send_raw(tensor, to_rank, lane)

    def send_raw(self, tensor: torch.Tensor, to_rank: int, lane: str) -> None:
        """Asynchronous header-less send (the receiver knows shape and dtype)."""
        payload = _wire_view(tensor.detach()).contiguous()
        work = dist.isend(payload, dst=dist.get_global_rank(self.pg, to_rank), group=lane_group(self.pg, lane))
        self._park(work, payload)

    def recv(self, from_rank: int, lane: str = FWD) -> Ticket:
        group = lane_group(self.pg, lane)
        src = dist.get_global_rank(self.pg, from_rank)
        pat = self._pattern("recv", from_rank, lane)
        if pat is not None and pat.frozen:
            if pat.pos >= len(pat.metas):
                raise RuntimeError(f"p2p static-shape contract broken from pipeline rank {from_rank} ({lane} lane): the micro-batch asks for tensor #{pat.pos} but the first one exchanged {len(pat.metas)}")
            meta = pat.metas[pat.pos]
        else:
            header = torch.empty(HEADER_LEN, dtype=torch.long, device=self.device)
            dist.recv(header, src=src, group=group)
            meta = P2PTensorMetaData.from_header(header)  # host read: only while shapes are unknown
            if pat is not None:
                pat.metas.append(meta)
        if pat is not None:
            pat.pos += 1
        buf = meta.create_empty_storage(self.device)
        work = dist.irecv(_wire_view(buf), src=src, group=group)
        return Ticket(buf, [work], meta.requires_grad)

    def recv_like(self, like: torch.Tensor, from_rank: int, lane: str) -> Ticket:
        """Post a header-less receive into a buffer shaped like ``like``."""
        buf = torch.empty(like.shape, dtype=like.dtype, device=self.device)
        work = dist.irecv(_wire_view(buf), src=dist.get_global_rank(self.pg, from_rank), group=lane_group(self.pg, lane))
        return Ticket(buf, [work], False)

    # ------------------------------------------------------------------ reference-style API (headers, forward lane)
    def _isend(self, tensor: torch.Tensor, to_rank: int, tag: int, static: Optional[bool] = None) -> List[dist.Work]:
        static = self._static if static is None else static
        meta = P2PTensorMetaData.from_tensor(tensor)
        group = lane_group(self.pg, FWD)
        dst = dist.get_global_rank(self.pg, to_rank)
        key = ("send", to_rank, tag)
        if not (static and self._tag_cache.get(key) == meta):
            if static and key in self._tag_cache:
                raise RuntimeError(f"p2p static-shape contract broken for peer {to_rank} tag {tag}: {self._tag_cache[key]} -> {meta}")
            dist.send(meta.to_header(self.device), dst=dst, group=group, tag=tag)
            if static:
                self._tag_cache[key] = meta
        payload = _wire_view(tensor.detach()).contiguous()
        work = dist.isend(payload, dst=dst, group=group, tag=tag)
        self._park(work, payload)
        return [work]

    def _irecv(self, from_rank: int, tag: int, static: Optional[bool] = None) -> Tuple[torch.Tensor, List[dist.Work]]:
        static = self._static if static is None else static
        group = lane_group(self.pg, FWD)
        src = dist.get_global_rank(self.pg, from_rank)
        key = ("recv", from_rank, tag)
        if static and key in self._tag_cache:
            meta = self._tag_cache[key]
        else:
            header = torch.empty(HEADER_LEN, dtype=torch.long, device=self.device)
            dist.recv(header, src=src, group=group, tag=tag)
            meta = P2PTensorMetaData.from_header(header)
            if static:
                self._tag_cache[key] = meta
        buf = meta.create_empty_storage(self.device)
        work = dist.irecv(_wire_view(buf), src=src, group=group, tag=tag)
        if meta.requires_grad:
            buf.requires_grad_(True)
        return buf, [work]

    def isend_tensors(self, tensors: List[torch.Tensor], to_rank: int, tag: int = 0, static: Optional[bool] = None) -> List[dist.Work]:
        """``static``: None follows ``expect_static``; False always sends the header (shapes that change from call to call)."""
        futures = []
        for t in tensors:
            futures.extend(self._isend(t, to_rank, tag, static))
        return futures

    def irecv_tensors(self, num_tensors: int, from_rank: int, tag: int = 0, static: Optional[bool] = None) -> Tuple[List[torch.Tensor], List[dist.Work]]:
        tensors, futures = [], []
        for _ in range(num_tensors):
            t, f = self._irecv(from_rank, tag, static)
            tensors.append(t)
            futures.extend(f)
        return tensors, futures

    def send_tensors(self, tensors: List[torch.Tensor], to_rank: int, tag: int = 0, static: Optional[bool] = None):
        for f in self.isend_tensors(tensors, to_rank, tag, static):
            f.wait()

    def recv_tensors(self, num_tensors: int, from_rank: int, tag: int = 0, static: Optional[bool] = None) -> List[torch.Tensor]:
        tensors, futures = self.irecv_tensors(num_tensors, from_rank, tag, static)
        for f in futures:
            f.wait()
        return tensors


class BatchTensorSendRecvState:
    """Queue sends and receives, then run them together (``flush``): all headers as one ``batch_isend_irecv``,
    then all payloads as another, so opposite-direction transfers cannot deadlock.  Used where no pipeline state is
    attached (plain forward calls across stages)."""

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
        group = lane_group(p2p.pg, FWD)
        peer = lambda r: dist.get_global_rank(p2p.pg, r)
        # phase 1: every header in one batched exchange (deadlock-free whatever the peer pattern)
        send_headers = [P2PTensorMetaData.from_tensor(t).to_header(p2p.device) for t, _ in self.send_queue]
        recv_headers = [torch.empty(HEADER_LEN, dtype=torch.long, device=p2p.device) for _ in self.recv_queue]
        hops = [dist.P2POp(dist.isend, h, peer(to), group=group) for h, (_, to) in zip(send_headers, self.send_queue)]
        hops += [dist.P2POp(dist.irecv, h, peer(frm), group=group) for h, frm in zip(recv_headers, self.recv_queue)]
        for w in dist.batch_isend_irecv(hops):
            w.wait()
        recv_meta = [P2PTensorMetaData.from_header(h) for h in recv_headers]
        # phase 2: payloads
        ops, bufs, keep = [], [], []
        for (t, to) in self.send_queue:
            payload = _wire_view(t.detach()).contiguous()
            keep.append(payload)
            ops.append(dist.P2POp(dist.isend, payload, peer(to), group=group))
        for meta, frm in zip(recv_meta, self.recv_queue):
            buf = meta.create_empty_storage(p2p.device)
            bufs.append((buf, meta))
            ops.append(dist.P2POp(dist.irecv, _wire_view(buf), peer(frm), group=group))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        out = []
        for buf, meta in bufs:
            if meta.requires_grad:
                buf.requires_grad_(True)
            out.append(buf)
        self._reset()
        return out
