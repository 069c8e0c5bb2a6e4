"""Compute + collective pairs of the tensor-parallel linears on CUDA.

``all_gather_matmul``: y = all_gather(x) @ W^T.  ``MatmulReduceScatter``: y = reduce_scatter(x @ W^T).

Fused path (``TPFusedContext``, needs the tp group inside one NVLink domain): buffers live in symmetric memory.
  all-gather -> GEMM : every rank pushes its block into slot `rank` of all peers' gather buffers with plain peer stores and
      raises a flag there; the tcgen05 GEMM's TMA producer (CTA-pair kernel by default) starts with the rows this rank wrote itself and polls the flag of
      a peer's block right before its first load from it, so the transfer of late blocks hides behind the math of early ones.
  GEMM -> reduce-scatter : the GEMM epilogue stores each bf16 tile of partial sums directly into the owner rank's staging
      slot (peer stores from registers), the last CTA raises a flag at every owner, and a small kernel sums the slots in
      fixed rank order (deterministic) once all flags are up.
Buffers and flags are double buffered; the stream order "signal for call c+1 comes after my kernels of call c" makes reuse
after two calls safe without extra barriers.  All waits are bounded.

Fallback path (any backend): NCCL collectives with the local block's GEMM issued first so it overlaps the transfer.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

import nanotron_b200.distributed as dist
from nanotron_b200.parallel.utils import MemoryBuffer

_CONTEXTS: Dict[int, Optional["TPFusedContext"]] = {}
ENABLED = True
# all-gather -> GEMM: True runs this rank's push on a side stream while the GEMM already works on the local rows (read from the
# pushed tensor itself); False (default) queues push, then GEMM, on one stream.  Measured on 2 x B200 (tp 2, Llama-3-8B): same
# bits, 0.653 ms against 0.644 ms for the [8192 x 4096] x [4096 x 14336] product and 38.3 k against 38.2 k tokens/s for the
# step: the push beside the GEMM costs the GEMM what it saves, so the single-stream order stays the default.
OVERLAP_PUSH = False


class TPFusedContext:
    """Symmetric buffers, flags and epochs for the fused tensor-parallel kernels of one process group."""

    def __init__(self, group):
        from nanotron_b200.parallel.symm import SymmetricAllocator

        self.group = group
        self.world = group.size()
        self.rank = dist.get_rank(group)
        self.alloc = SymmetricAllocator(group)
        dev = self.alloc.device
        self.gather = [None, None]
        self.staging = [None, None]
        self.ag_flags = [self.alloc.zeros(32, torch.int32) for _ in range(2)]
        self.rs_flags = [self.alloc.zeros(32, torch.int32) for _ in range(2)]
        self.ag_calls = 0
        self.rs_calls = 0
        self.ce_calls = 0
        self.ce_parts = [None, None]
        self.counter = torch.zeros(4, dtype=torch.int32, device=dev)
        self.status = self.alloc.status
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.side = torch.cuda.Stream(device=dev, priority=-1)  # pushes that overlap their GEMM; high priority so its small CTAs are placed first

    # ---- vocabulary-parallel cross entropy: (max, sum exp, target logit) combined by peer loads
    def ce_combine(self, local_max: torch.Tensor, local_sumexp: torch.Tensor, local_tgt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (logZ, loss) per row from every rank's partial statistics; no NCCL collective."""
        from nanotron_b200.ops import native

        rows = local_max.numel()
        i = self.ce_calls & 1
        self.ce_calls += 1
        cur = self.ce_parts[i]
        if cur is None or cur.tensor.numel() < 3 * rows:
            cur = self.ce_parts[i] = self.alloc.zeros(3 * rows, torch.float32)  # collective: same size on every rank
        pitch = cur.tensor.numel() // 3
        view = cur.tensor.view(3, pitch)
        view[0, :rows].copy_(local_max)
        view[1, :rows].copy_(local_sumexp)
        view[2, :rows].copy_(local_tgt)
        self.alloc.barrier()  # every rank's triple is in place (the other parity buffer may still be read by a slow peer)
        logz = torch.empty(rows, dtype=torch.float32, device=local_max.device)
        loss = torch.empty_like(logz)
        L = native.lib()
        L.ntb_ce_combine_peers.restype = ctypes.c_int
        L.ntb_ce_combine_peers.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        rc = L.ntb_ce_combine_peers(cur.ptrs, self.world, rows, pitch, logz.data_ptr(), loss.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "ce_combine_peers")
        return logz, loss

    @staticmethod
    def _entry(kind: str):
        """The fused GEMMs exist on both in-tree GEMM kernels; the CTA-pair kernel (the default of ``native_gemm``) is the faster one."""
        from nanotron_b200.ops import native, native_gemm

        L = native.lib()
        pair = native_gemm.VARIANT["kernel"] == "pair" and hasattr(L, "ntb_gemm2_bf16_ag")
        return getattr(L, ("ntb_gemm2_bf16_" if pair else "ntb_gemm_bf16_") + kind)

    def _buf(self, pool, i: int, numel: int):
        cur = pool[i]
        if cur is None or cur.tensor.numel() < numel:
            pool[i] = self.alloc.zeros(numel, torch.bfloat16)  # collective: every rank asks for the same size at the same call
        return pool[i]

    # ---- all-gather (optionally fused with the GEMM that consumes it)
    def push(self, x2: torch.Tensor, stream: Optional["torch.cuda.Stream"] = None) -> Tuple[torch.Tensor, "object", int, int]:
        """Copies x2 into slot `rank` of every rank's gather buffer and raises the flags; on `stream` (after everything the
        current stream has queued so far) when given, else on the current stream."""
        from nanotron_b200.ops import native

        M, K = x2.shape
        i = self.ag_calls & 1
        self.ag_calls += 1
        epoch = self.ag_calls
        buf = self._buf(self.gather, i, self.world * M * K)  # (re)allocation is a collective on the current stream
        flags = self.ag_flags[i]
        main = torch.cuda.current_stream()
        if stream is not None:
            ready = torch.cuda.Event()
            ready.record(main)  # x2 is complete, and every earlier reader of this gather buffer is done
            stream.wait_event(ready)
        rc = native.lib().ntb_tp_allgather_push(x2.data_ptr(), buf.ptrs, flags.ptrs, self.rank, self.world, M * K, epoch, self.counter[0:1].data_ptr(), (stream or main).cuda_stream)
        native._check(rc, "tp_allgather_push")
        gathered = buf.tensor[: self.world * M * K].view(self.world * M, K)
        return gathered, flags, epoch, M

    def wait(self, flags, epoch: int):
        from nanotron_b200.ops import native

        rc = native.lib().ntb_symm_wait(flags.tensor.data_ptr(), self.world, epoch, self.alloc.wait_limit_ns, self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "symm_wait")

    def all_gather_gemm(self, x2: torch.Tensor, weight: torch.Tensor, b_mn: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        """out = gather(x2) @ W^T (b_mn False, W [N, K]) or gather(x2) @ W (b_mn True, W [K, N])."""
        from nanotron_b200.ops import native, native_gemm

        L = native.lib()
        N = weight.shape[1] if b_mn else weight.shape[0]
        K = x2.shape[1]
        main = torch.cuda.current_stream()
        local = OVERLAP_PUSH and self.world > 1 and native_gemm.VARIANT["kernel"] == "pair" and hasattr(L, "ntb_gemm2_bf16_ag_local")
        gathered, flags, epoch, M = self.push(x2, stream=self.side if local else None)
        out = torch.empty((self.world * M, N), dtype=x2.dtype, device=x2.device)
        native_gemm.ensure_workspace(x2.device)
        tail = (self.world * M, N, K, K, weight.stride(0), N, int(b_mn), flags.tensor.data_ptr(), M, self.rank, self.world, epoch, self.status.data_ptr(), self.sms, main.cuda_stream)
        if local:
            # the GEMM reads its own rows from x2, so it depends on no kernel of this GPU: the push runs beside it
            rc = L.ntb_gemm2_bf16_ag_local(gathered.data_ptr(), x2.data_ptr(), x2.stride(0), weight.data_ptr(), out.data_ptr(), *tail)
            pushed = torch.cuda.Event()
            pushed.record(self.side)
            main.wait_event(pushed)  # later readers of `gathered` (wgrad) and the next owner of x2's memory come after the push
        else:
            rc = self._entry("ag")(gathered.data_ptr(), weight.data_ptr(), out.data_ptr(), *tail)
        native._check(rc, "gemm_bf16_ag")
        return out, gathered

    def gemm_reduce_scatter(self, x2: torch.Tensor, weight: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """out[M/tp, N] = reduce_scatter(x2 @ W^T) (or x2 @ W when b_mn)."""
        from nanotron_b200.ops import native

        M, K = x2.shape
        N = weight.shape[1] if b_mn else weight.shape[0]
        rows = M // self.world
        i = self.rs_calls & 1
        self.rs_calls += 1
        epoch = self.rs_calls
        buf = self._buf(self.staging, i, self.world * rows * N)
        flags = self.rs_flags[i]
        L = native.lib()
        stream = torch.cuda.current_stream().cuda_stream
        rc = self._entry("rs")(x2.data_ptr(), weight.data_ptr(), M, N, K, x2.stride(0), weight.stride(0), int(b_mn), buf.ptrs, flags.ptrs, rows, self.rank, self.world, epoch, self.counter[1:2].data_ptr(), self.status.data_ptr(), self.sms, stream)
        native._check(rc, "gemm_bf16_rs")
        out = torch.empty((rows, N), dtype=x2.dtype, device=x2.device)
        rc = L.ntb_tp_reduce_slots(buf.tensor.data_ptr(), out.data_ptr(), flags.tensor.data_ptr(), self.world, rows * N, epoch, self.alloc.wait_limit_ns, self.status.data_ptr(), stream)
        native._check(rc, "tp_reduce_slots")
        return out


def get_context(group) -> Optional[TPFusedContext]:
    key = id(group)
    if key not in _CONTEXTS:
        ctx = None
        try:
            from nanotron_b200 import ops
            from nanotron_b200.parallel import symm

            if ENABLED and ops.get_mode() != "torch" and group.size() <= 8 and symm.is_available(group):
                ctx = TPFusedContext(group)
        except Exception as e:  # symmetric memory not usable for this group (e.g. spans nodes)
            import warnings

            warnings.warn(f"fused tensor-parallel kernels disabled for this group, using NCCL: {type(e).__name__}: {e}")
            ctx = None
        _CONTEXTS[key] = ctx
    return _CONTEXTS[key]


def _fusable(x2: torch.Tensor, weight: torch.Tensor, rows_per_rank: int) -> bool:
    from nanotron_b200 import ops

    if ops.get_linear() == "fp8":
        return False  # the fused kernels are bf16: fp8 products take the collective + local fp8 GEMM route
    return (
        x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x2.is_contiguous() and weight.is_contiguous()
        and rows_per_rank % 128 == 0 and x2.shape[1] % 64 == 0 and weight.shape[0] % 64 == 0 and weight.shape[1] % 64 == 0
    )


def all_gather_matmul(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group, keep_gathered: bool, lead_rows: int) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (y[tp*M, N], gathered x or None).  Rows of rank r land at [r*M, (r+1)*M)."""
    from nanotron_b200 import ops

    tp = group.size()
    rank = dist.get_rank(group)
    M, K = x2.shape
    x2 = x2.contiguous()
    ctx = get_context(group) if x2.is_cuda else None
    if ctx is not None and _fusable(x2, weight, M):
        out, gathered = ctx.all_gather_gemm(x2, weight, b_mn=False)
        if bias is not None:
            out = out + bias
        return out, (gathered.clone() if keep_gathered else None)
    if keep_gathered:
        gathered = torch.empty((tp * M, K), dtype=x2.dtype, device=x2.device)
    else:
        gathered = MemoryBuffer().get("allgather", (tp * M, K), dtype=x2.dtype, device=x2.device)
    out = torch.empty((tp * M, weight.shape[0]), dtype=x2.dtype, device=x2.device)
    handle = dist.all_gather_into_tensor(gathered, x2, group=group, async_op=True)
    # local shard first: its GEMM hides the transfer of the remote shards
    out[rank * M : (rank + 1) * M] = ops.linear_forward(x2, weight, bias)
    handle.wait()
    if rank > 0:
        out[: rank * M] = ops.linear_forward(gathered[: rank * M], weight, bias)
    if rank < tp - 1:
        out[(rank + 1) * M :] = ops.linear_forward(gathered[(rank + 1) * M :], weight, bias)
    return out, (gathered if keep_gathered else None)


class MatmulReduceScatter(torch.autograd.Function):
    """out[M/tp, N] = reduce_scatter_dim0(x[M, K_local] @ W[N, K_local]^T); backward all-gathers dY and runs the dgrad on it
    (fused all-gather -> GEMM when available) (parity: reference functional.py:569-695)."""

    @staticmethod
    def forward(ctx, x, weight, group):
        from nanotron_b200 import ops

        tp = group.size()
        ctx.group = group
        ctx.save_for_backward(x, weight)
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        assert M % tp == 0
        fctx = get_context(group) if x2.is_cuda else None
        if fctx is not None and _fusable(x2.contiguous(), weight, M // tp):
            out = fctx.gemm_reduce_scatter(x2.contiguous(), weight, b_mn=False)
        else:
            out = torch.empty((M // tp, weight.shape[0]), dtype=x.dtype, device=x.device)
            full = ops.linear_forward(x2, weight, None)
            dist.reduce_scatter_tensor(out, full, group=group)
        return out.view(x.shape[0] // tp, *x.shape[1:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        from nanotron_b200 import ops

        x, weight = ctx.saved_tensors
        group = ctx.group
        tp = group.size()
        go = grad_output.contiguous()
        go2 = go.reshape(-1, go.shape[-1])
        fctx = get_context(group) if go.is_cuda else None
        if fctx is not None and _fusable(go2, weight, go2.shape[0]) and ctx.needs_input_grad[0]:
            gi2, total2 = fctx.all_gather_gemm(go2, weight, b_mn=True)
            grad_input = gi2.view(x.shape)
            # every block has arrived once the gated GEMM finished: the wgrad may read the gathered buffer directly
            grad_weight = ops.linear_wgrad(total2, x.reshape(-1, x.shape[-1]), weight)
            return grad_input, grad_weight, None
        total = MemoryBuffer().get("allgather2", (go.shape[0] * tp, *go.shape[1:]), dtype=go.dtype, device=go.device)
        dist.all_gather_into_tensor(total, go, group=group)
        total2 = total.reshape(-1, total.shape[-1])
        grad_input = ops.linear_dgrad(total2, weight).view(x.shape) if ctx.needs_input_grad[0] else None
        grad_weight = ops.linear_wgrad(total2, x.reshape(-1, x.shape[-1]), weight)
        return grad_input, grad_weight, None


def fused_all_gather(x2: torch.Tensor, group) -> Optional[torch.Tensor]:
    """All-gather on dim 0 through the push kernel (returns a view of a symmetric buffer valid until two calls later),
    or None when the fused path does not apply."""
    ctx = get_context(group) if x2.is_cuda else None
    if ctx is None or x2.dtype != torch.bfloat16 or (x2.numel() % 8) or not x2.is_contiguous():
        return None
    gathered, flags, epoch, _ = ctx.push(x2)
    ctx.wait(flags, epoch)
    return gathered


def fused_matmul_reduce_scatter(go2: torch.Tensor, weight: torch.Tensor, group, b_mn: bool) -> Optional[torch.Tensor]:
    ctx = get_context(group) if go2.is_cuda else None
    if ctx is None or not _fusable(go2, weight, go2.shape[0] // group.size()):
        return None
    return ctx.gemm_reduce_scatter(go2, weight, b_mn=b_mn)
