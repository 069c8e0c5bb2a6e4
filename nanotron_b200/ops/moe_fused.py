"""Expert-parallel mixture-of-experts MLP on the in-tree kernels: device-side routing plan, token dispatch / combine over
NVLink peer memory, and tcgen05 grouped GEMMs (``csrc/moe_dispatch.cu``, ``csrc/gemm_tcgen05.cu``).

Nothing here synchronises with the host: counts, offsets and the number of used row blocks stay on the device, so the
launch sequence of a layer does not depend on the routing.  (The reference moves the per-expert batch sizes to the CPU for
its grouped GEMM, src/nanotron/nn/moe.py:93, and has no expert-parallel communication at all.)

``fused_moe_experts(x, top_p, top_i, counts, w_gate_up, w_down, group)`` is differentiable in ``x``, ``top_p`` and the two
weights.  With ``group`` of size 1 (or None) the same kernels run on local buffers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p
from typing import Dict, Optional, Tuple

import torch

from nanotron_b200 import distributed as dist
from nanotron_b200.ops import native

_CONTEXTS: Dict[Tuple[int, int, int, int], "MoEContext"] = {}
_DECLARED = False


def _lib():
    global _DECLARED
    L = native.lib()
    if not _DECLARED:
        c_u32, c_ull = ctypes.c_uint32, ctypes.c_ulonglong
        L.ntb_gemm_bf16_grouped.restype = c_int
        L.ntb_gemm_bf16_grouped.argtypes = [c_void_p] * 3 + [c_int] * 5 + [c_void_p] * 3 + [c_int, c_void_p]
        L.ntb_gemm_bf16_grouped_wgrad.restype = c_int
        L.ntb_gemm_bf16_grouped_wgrad.argtypes = [c_void_p] * 3 + [c_int] * 4 + [c_void_p, c_int, c_void_p, c_int, c_void_p]
        L.ntb_moe_plan.restype = c_int
        L.ntb_moe_plan.argtypes = [c_void_p] * 3 + [c_int] * 3 + [c_u32, c_ull] + [c_void_p] * 6 + [c_int, c_void_p]
        L.ntb_moe_rank.restype = c_int
        L.ntb_moe_rank.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]
        L.ntb_moe_dispatch.restype = c_int
        L.ntb_moe_dispatch.argtypes = [c_void_p] * 6 + [c_int] * 5 + [c_void_p]
        L.ntb_moe_zero_pad.restype = c_int
        L.ntb_moe_zero_pad.argtypes = [c_void_p] * 3 + [c_int, c_int, c_void_p]
        L.ntb_moe_combine.restype = c_int
        L.ntb_moe_combine.argtypes = [c_void_p] * 7 + [c_int] * 5 + [c_void_p]
        L.ntb_moe_scale_dot.restype = c_int
        L.ntb_moe_scale_dot.argtypes = [c_void_p] * 8 + [c_int, c_int, c_void_p]
        _DECLARED = True
    return L


def available() -> bool:
    return native.available() and hasattr(native.lib(), "ntb_moe_plan")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Plan:
    """Device-side description of one routing: everything the grouped GEMMs and the combine need."""

    __slots__ = ("seg_off", "cnt_tot", "dest_base", "tile_expert", "num_m_tiles", "row_of")


class MoEContext:
    """Receive / result buffers (peer-addressable when the group has more than one rank), flags and epochs."""

    def __init__(self, group, hidden: int, cap_rows: int, num_experts: int):
        self.group = group
        self.world = group.size() if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.hidden, self.cap_rows, self.num_experts = hidden, cap_rows, num_experts
        self.local_experts = num_experts // self.world
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.epoch = 0
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        if self.world > 1:
            from nanotron_b200.parallel.symm import SymmetricAllocator

            self.alloc = SymmetricAllocator(group)
            mk = lambda n, dt: self.alloc.zeros(n, dt)  # noqa: E731
            self.status = self.alloc.status
            self.limit_ns = self.alloc.wait_limit_ns
        else:
            self.alloc = None
            mk = lambda n, dt: _LocalTensor(torch.zeros(n, dtype=dt, device=self.device))  # noqa: E731
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.limit_ns = 2_000_000_000
        self.recv = mk(cap_rows * hidden, torch.bfloat16)
        self.ybuf = mk(cap_rows * hidden, torch.bfloat16)
        self.p_recv = mk(cap_rows, torch.float32)
        self.dp_rows = mk(cap_rows, torch.float32)
        self.tables = mk(2 * self.world * num_experts, torch.int32)
        self.plan_flags = mk(32, torch.int32)

    # ---- building blocks
    def barrier(self):
        if self.alloc is not None:
            self.alloc.barrier()

    def check(self):
        v = int(self.status.item())
        if v != 0:
            self.status.zero_()
            raise native.NativeKernelError(f"mixture-of-experts exchange failed with status {v} (1 = routing exceeded the buffer, 3 = a peer did not answer in time)")

    def make_plan(self, counts: torch.Tensor, top_i: torch.Tensor) -> Plan:
        L = _lib()
        p = Plan()
        El, E = self.local_experts, self.num_experts
        cap_tiles = self.cap_rows // 128
        i32 = dict(dtype=torch.int32, device=self.device)
        p.seg_off = torch.empty(El + 1, **i32)
        p.cnt_tot = torch.empty(El, **i32)
        p.dest_base = torch.empty(E, **i32)
        p.tile_expert = torch.zeros(cap_tiles, **i32)
        p.num_m_tiles = torch.empty(1, **i32)
        p.row_of = torch.empty(top_i.numel(), **i32)
        self.epoch += 1
        rc = L.ntb_moe_plan(counts.data_ptr(), self.tables.ptrs, self.plan_flags.ptrs, self.rank, self.world, E, self.epoch, self.limit_ns, self.status.data_ptr(),
                            p.seg_off.data_ptr(), p.cnt_tot.data_ptr(), p.dest_base.data_ptr(), p.tile_expert.data_ptr(), p.num_m_tiles.data_ptr(), cap_tiles, _stream())
        native._check(rc, "moe_plan")
        rc = L.ntb_moe_rank(top_i.data_ptr(), top_i.numel(), p.dest_base.data_ptr(), E, p.row_of.data_ptr(), _stream())
        native._check(rc, "moe_rank")
        return p

    def dispatch(self, x: torch.Tensor, top_i: torch.Tensor, plan: Plan, top_p: Optional[torch.Tensor], zero_pad: bool):
        """Rows of ``x`` -> the owners' ``recv`` (and ``top_p`` -> ``p_recv``); returns after the cross-rank barrier is enqueued."""
        L = _lib()
        T, h = x.shape
        k = top_i.shape[1]
        rc = L.ntb_moe_dispatch(x.data_ptr(), top_i.data_ptr(), plan.row_of.data_ptr(), top_p.data_ptr() if top_p is not None else None, self.recv.ptrs,
                                self.p_recv.ptrs if top_p is not None else None, T, h, k, self.world, self.num_experts, _stream())
        native._check(rc, "moe_dispatch")
        if zero_pad:
            rc = L.ntb_moe_zero_pad(self.recv.tensor.data_ptr(), plan.seg_off.data_ptr(), plan.cnt_tot.data_ptr(), h, self.local_experts, _stream())
            native._check(rc, "moe_zero_pad")
        self.barrier()

    def combine(self, top_i: torch.Tensor, plan: Plan, weights: Optional[torch.Tensor], T: int, gather_scalars: bool):
        L = _lib()
        k = top_i.shape[1]
        out = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        scal = torch.empty((T, k), dtype=torch.float32, device=self.device) if gather_scalars else None
        rc = L.ntb_moe_combine(self.ybuf.ptrs, top_i.data_ptr(), plan.row_of.data_ptr(), weights.data_ptr() if weights is not None else None, out.data_ptr(),
                               self.dp_rows.ptrs if gather_scalars else None, scal.data_ptr() if gather_scalars else None, T, self.hidden, k, self.world,
                               self.num_experts, _stream())
        native._check(rc, "moe_combine")
        return out, scal

    def grouped(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool, plan: Plan, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a [cap, K] times w[e]: b_mn -> w is [E, K, N]; else w is [E, N, K]."""
        L = _lib()
        cap, K = a.shape
        N = w.shape[2] if b_mn else w.shape[1]
        assert (w.shape[1] if b_mn else w.shape[2]) == K and w.is_contiguous() and a.is_contiguous()
        if out is None:
            out = torch.empty((cap, N), dtype=torch.bfloat16, device=a.device)
        rc = L.ntb_gemm_bf16_grouped(a.data_ptr(), w.data_ptr(), out.data_ptr(), cap, N, K, int(b_mn), w.shape[0], plan.tile_expert.data_ptr(),
                                     plan.num_m_tiles.data_ptr(), self.status.data_ptr(), self.sms, _stream())
        native._check(rc, "gemm_bf16_grouped")
        return out

    def grouped_wgrad(self, x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor, plan: Plan) -> Optional[torch.Tensor]:
        """dW[e] = x_e^T dy_e, accumulated into ``weight.main_grad`` (fp32) when present, else returned in bf16."""
        L = _lib()
        cap, M = x.shape
        N = dy.shape[1]
        E = weight.shape[0]
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            dst, mode, ret = main_grad, 2, None
        else:
            dst = torch.zeros((E, M, N), dtype=torch.bfloat16, device=x.device)
            mode, ret = 0, dst
        rc = L.ntb_gemm_bf16_grouped_wgrad(x.data_ptr(), dy.data_ptr(), dst.data_ptr(), cap, M, N, E, plan.seg_off.data_ptr(), mode, self.status.data_ptr(), self.sms, _stream())
        native._check(rc, "gemm_bf16_grouped_wgrad")
        return ret

    def scale_dot(self, y_saved: torch.Tensor, plan: Plan):
        L = _lib()
        rc = L.ntb_moe_scale_dot(self.recv.tensor.data_ptr(), y_saved.data_ptr(), self.p_recv.tensor.data_ptr(), self.dp_rows.tensor.data_ptr(), plan.num_m_tiles.data_ptr(),
                                 plan.tile_expert.data_ptr(), plan.seg_off.data_ptr(), plan.cnt_tot.data_ptr(), self.hidden, self.cap_rows, _stream())
        native._check(rc, "moe_scale_dot")


class _LocalTensor:
    """Single-rank stand-in for a symmetric tensor: the peer table holds the tensor's own address."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor
        self.ptrs = (ctypes.c_uint64 * 1)(tensor.data_ptr())


def capacity_rows(tokens: int, top_k: int, world: int, local_experts: int) -> int:
    """Worst case (every assignment of every rank lands on this rank) plus one padding block per local expert."""
    return ((world * tokens * top_k + 127) // 128) * 128 + local_experts * 128


def get_context(group, hidden: int, tokens: int, top_k: int, num_experts: int) -> MoEContext:
    world = group.size() if group is not None else 1
    cap = capacity_rows(tokens, top_k, world, num_experts // world)
    key = (id(group) if group is not None else 0, hidden, cap, num_experts)
    if key not in _CONTEXTS:
        _CONTEXTS[key] = MoEContext(group, hidden, cap, num_experts)
    return _CONTEXTS[key]


def supported(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, num_experts: int, top_k: int, group) -> bool:
    world = group.size() if group is not None else 1
    h, two_i = w_gate_up.shape[1], w_gate_up.shape[2]
    return (
        x.is_cuda and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16 and available()
        and h % 64 == 0 and two_i % 128 == 0 and num_experts <= 256 and top_k <= 16 and world <= 8 and num_experts % world == 0
    )


class _FusedMoEExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, top_p, top_i, counts, w_gate_up, w_down, mctx: MoEContext):
        T, h = x.shape
        x = x.contiguous()
        top_p = top_p.contiguous().float()
        top_i = top_i.contiguous()
        plan = mctx.make_plan(counts.to(torch.int32).contiguous(), top_i)
        mctx.dispatch(x, top_i, plan, None, zero_pad=True)
        recv = mctx.recv.tensor.view(mctx.cap_rows, h)
        x_perm = recv.clone()
        gu = mctx.grouped(x_perm, w_gate_up, True, plan)
        a = native.swiglu_fwd(gu)
        ybuf = mctx.ybuf.tensor.view(mctx.cap_rows, h)
        mctx.grouped(a, w_down, True, plan, out=ybuf)
        del a
        y_saved = ybuf.clone() if (x.requires_grad or top_p.requires_grad or w_down.requires_grad) else None
        mctx.barrier()
        out, _ = mctx.combine(top_i, plan, top_p, T, gather_scalars=False)
        ctx.mctx, ctx.plan = mctx, plan
        ctx.w_gate_up, ctx.w_down = w_gate_up, w_down  # kept as objects: their fp32 main_grad attribute is needed in backward
        ctx.save_for_backward(top_p, top_i, x_perm, gu, y_saved)
        return out

    @staticmethod
    def backward(ctx, d_out):
        mctx, plan = ctx.mctx, ctx.plan
        top_p, top_i, x_perm, gu, y_saved = ctx.saved_tensors
        w_gate_up, w_down = ctx.w_gate_up, ctx.w_down
        T, h = d_out.shape
        d_out = d_out.contiguous()
        mctx.dispatch(d_out, top_i, plan, top_p, zero_pad=False)
        mctx.scale_dot(y_saved, plan)  # recv <- p * dOut rows (padding zero); dp_rows <- <dOut row, Y row>
        dy_perm = mctx.recv.tensor.view(mctx.cap_rows, h)
        a = native.swiglu_fwd(gu)
        d_w_down = mctx.grouped_wgrad(a, dy_perm, w_down, plan)
        del a
        d_a = mctx.grouped(dy_perm, w_down, False, plan)  # w_down [E, I, h] read as [E, N = I, K = h]
        d_gu = native.swiglu_bwd(gu, d_a)
        del d_a
        d_w_gate_up = mctx.grouped_wgrad(x_perm, d_gu, w_gate_up, plan)
        ybuf = mctx.ybuf.tensor.view(mctx.cap_rows, h)
        mctx.grouped(d_gu, w_gate_up, False, plan, out=ybuf)  # w_gate_up [E, h, 2I] read as [E, N = h, K = 2I]
        mctx.barrier()
        dx, d_top_p = mctx.combine(top_i, plan, None, T, gather_scalars=True)
        return dx, d_top_p, None, None, d_w_gate_up, d_w_down, None


def fused_moe_experts(x, top_p, top_i, counts, w_gate_up, w_down, group=None) -> torch.Tensor:
    num_experts = w_gate_up.shape[0] * (group.size() if group is not None else 1)
    mctx = get_context(group, x.shape[1], x.shape[0], top_i.shape[1], num_experts)
    return _FusedMoEExperts.apply(x, top_p, top_i, counts, w_gate_up, w_down, mctx)
