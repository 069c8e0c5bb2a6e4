"""Hot ops of the framework.

Each op has two implementations: the in-tree sm_100a CUDA kernel (``nanotron_b200.ops.native``, C ABI in
``csrc/``) used for CUDA tensors, and the PyTorch fp32 oracle (``nanotron_b200.ops.reference``) used on CPU and
in tests.  On a CUDA device a missing extension is an error, never a silent fallback; the oracle can be forced
with ``ops.set_mode("torch")``.
"""
from __future__ import annotations

import math
import os
from contextlib import contextmanager
from typing import Optional, Tuple

import torch

from nanotron_b200.ops import reference as ref

_MODE = os.environ.get("NTB_OPS", "auto")  # auto | torch
_GEMM = os.environ.get("NTB_GEMM", "auto")  # auto | cublas | tcgen05
_ATTN = os.environ.get("NTB_ATTN", "auto")  # auto | native (both: the in-tree tcgen05 kernels) | sdpa (library kernel, for comparison)
_LINEAR = os.environ.get("NTB_LINEAR", "bf16")  # bf16 | fp8 (block-scaled e4m3 forward / e5m2 gradients for the linear-layer products)
LAUNCH_COUNTER = {"n": 0}


def set_mode(mode: str):
    global _MODE
    assert mode in ("auto", "torch")
    _MODE = mode


def set_gemm(mode: str):
    global _GEMM
    assert mode in ("auto", "cublas", "tcgen05")
    _GEMM = mode


def set_attention(mode: str):
    global _ATTN
    assert mode in ("auto", "native", "sdpa")
    _ATTN = mode


def set_linear(mode: str):
    """Operand precision of the three products of every tensor-parallel linear layer: "bf16", or "fp8" = block-scaled fp8
    (1 x 128 activation / gradient blocks, 128 x 128 weight blocks, e4m3 forward, e5m2 gradients; ``nanotron_b200.fp8``).  Products
    whose shapes are not multiples of 128 (the padded lm head shard, toy models) stay in bf16."""
    global _LINEAR
    assert mode in ("bf16", "fp8")
    _LINEAR = mode


def get_linear() -> str:
    return _LINEAR


def get_mode() -> str:
    return _MODE


@contextmanager
def mode(m: str):
    global _MODE
    old = _MODE
    set_mode(m)
    try:
        yield
    finally:
        _MODE = old


def native_launches() -> int:
    """Number of in-tree kernel launches issued by this process so far."""
    return LAUNCH_COUNTER["n"]


def _use_native(t: torch.Tensor) -> bool:
    if _MODE == "torch" or not t.is_cuda:
        return False
    from nanotron_b200.ops import native

    native.lib()  # raises when the extension is missing: no silent fallback on GPU
    return True


# ============================================================================ GEMM
def _tcgen05_ok(a: torch.Tensor, b: torch.Tensor, kind: str) -> bool:
    """Which GEMMs run on the in-tree tcgen05 kernels.  "auto": every linear-layer product (forward, dgrad, wgrad with or without
    fp32 accumulation) whose operands the kernels accept and that is large enough to fill the GPU; small or oddly shaped
    products go to the library.  "tcgen05": the same without the size threshold.  "cublas": nothing (comparison runs)."""
    if _GEMM == "cublas" or not a.is_cuda or _MODE == "torch":
        return False
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return False
    from nanotron_b200.ops import native

    return native.gemm_supported(a, b, force=_GEMM == "tcgen05")


def linear_forward(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[M,N] = x2[M,K] @ weight[N,K]^T (+ bias)."""
    if _LINEAR == "fp8":
        from nanotron_b200.fp8 import linear as fp8_linear

        if fp8_linear.shapes_ok(x2, weight):
            y = fp8_linear.fp8_forward(x2, weight)
            return y if bias is None else y + bias
    if _tcgen05_ok(x2, weight, "fwd"):
        from nanotron_b200.ops import native

        y = native.gemm_nt(x2, weight)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x2, weight, bias)


def linear_dgrad(go2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """dx[M,K] = go2[M,N] @ weight[N,K]."""
    if _LINEAR == "fp8":
        from nanotron_b200.fp8 import linear as fp8_linear

        if fp8_linear.shapes_ok(go2, weight.t()):
            return fp8_linear.fp8_dgrad(go2, weight)
    if _tcgen05_ok(go2, weight, "dgrad"):
        from nanotron_b200.ops import native

        return native.gemm_nn(go2, weight)
    return go2.matmul(weight)


def linear_wgrad(go2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """dW[N,K] = go2[M,N]^T @ x2[M,K].  When the weight carries an fp32 ``main_grad`` buffer the product is
    accumulated into it and ``None`` is returned (autograd then leaves ``weight.grad`` unset)."""
    main_grad = getattr(weight, "main_grad", None)
    if _LINEAR == "fp8":
        from nanotron_b200.fp8 import linear as fp8_linear

        if fp8_linear.shapes_ok(x2, weight) and go2.shape[0] % 128 == 0:
            return fp8_linear.fp8_wgrad(go2, x2, weight)
    if main_grad is not None:
        if _tcgen05_ok(go2, x2, "wgrad_accum"):
            from nanotron_b200.ops import native

            native.gemm_tn_accum_fp32(go2, x2, main_grad)
        else:
            gw = go2.t().matmul(x2)
            main_grad.add_(gw)
        return None
    if _tcgen05_ok(go2, x2, "wgrad"):
        from nanotron_b200.ops import native

        return native.gemm_tn(go2, x2)
    return go2.t().matmul(x2)


# ============================================================================ embedding
class _MaskedEmbedding(torch.autograd.Function):
    """Vocabulary-range-masked lookup; the weight gradient goes straight into the fp32 ``main_grad`` buffer when there is one
    (parity: reference tensor_parallel/nn.py:275-301 masks the ids, looks up, then masks the output again)."""

    @staticmethod
    def forward(ctx, ids, weight, min_id, max_id):
        from nanotron_b200.ops import native

        ctx.save_for_backward(ids, weight)
        ctx.range = (min_id, max_id)
        return native.embedding_fwd(ids, weight, min_id, max_id)

    @staticmethod
    def backward(ctx, dout):
        from nanotron_b200.ops import native

        ids, weight = ctx.saved_tensors
        min_id, max_id = ctx.range
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            native.embedding_bwd_accum(ids, dout, main_grad, min_id, max_id)
            return None, None, None, None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        native.embedding_bwd_accum(ids, dout, dw, min_id, max_id)
        return None, dw.to(weight.dtype), None, None


def masked_embedding(ids: torch.Tensor, weight: torch.Tensor, min_id: int, max_id: int) -> torch.Tensor:
    """Rows of ``weight`` ([max_id - min_id, h]) for ids inside [min_id, max_id), zeros for the others."""
    if _use_native(weight) and ids.dtype == torch.int64 and weight.is_contiguous() and (weight.shape[1] * weight.element_size()) % 16 == 0 and weight.shape[1] % 8 == 0:
        return _MaskedEmbedding.apply(ids, weight, min_id, max_id)
    mask = (ids < min_id) | (ids >= max_id)
    out = torch.nn.functional.embedding((ids - min_id).masked_fill(mask, 0), weight)
    return out.masked_fill(mask.unsqueeze(-1), 0.0)


# ============================================================================ norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual, passthrough=False):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, shape[-1]) if residual is not None else None
        if _use_native(x):
            from nanotron_b200.ops import native

            y, pre, rstd = native.rmsnorm_fwd(x2.contiguous(), r2.contiguous() if r2 is not None else None, weight, eps)
        else:
            y, pre, rstd = ref.rms_norm_fwd(x2, weight, eps, r2)
        ctx.save_for_backward(pre, weight, rstd)
        ctx.has_residual = residual is not None
        ctx.shape = shape
        if residual is not None:
            return y.view(shape), pre.view(shape)
        if passthrough:
            # the input comes back as a second output, so the gradient of its other consumers arrives here as ``dpre`` and the
            # backward kernel adds it while it writes dx (no separate accumulation kernel in autograd)
            return y.view(shape), x
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dpre):
        pre, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, ctx.shape[-1]).contiguous()
        dres = dpre.reshape(-1, ctx.shape[-1]).contiguous() if dpre is not None else None
        if _use_native(dy2):
            from nanotron_b200.ops import native

            dx, dw = native.rmsnorm_bwd(dy2, pre, weight, rstd, dres)
        else:
            dx, dw = ref.rms_norm_bwd(dy2, pre, weight, rstd, dres)
        dx = dx.view(ctx.shape)
        return dx, dw.to(weight.dtype), None, (dx if ctx.has_residual else None), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None, return_input: bool = False):
    """Returns ``y`` (no residual) or ``(y, x + residual)``: the fused residual-add + norm used between blocks.
    ``return_input`` (without a residual) returns ``(y, x)`` where the second output stands for ``x`` in the rest of the graph: use
    it for the skip connection and the sum of the two gradient paths is fused into the norm's backward kernel."""
    y, pre = _RMSNorm.apply(x, weight, eps, residual, return_input and residual is None)
    return y if (residual is None and not return_input) else (y, pre)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, shape[-1]) if residual is not None else None
        if _use_native(x):
            from nanotron_b200.ops import native

            y, pre, mean, rstd = native.layernorm_fwd(x2.contiguous(), r2.contiguous() if r2 is not None else None, weight, bias, eps)
        else:
            y, pre, mean, rstd = ref.layer_norm_fwd(x2, weight, bias, eps, r2)
        ctx.save_for_backward(pre, weight, mean, rstd)
        ctx.has_residual, ctx.has_bias, ctx.shape = residual is not None, bias is not None, shape
        return y.view(shape), (pre.view(shape) if residual is not None else None)

    @staticmethod
    def backward(ctx, dy, dpre):
        pre, weight, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, ctx.shape[-1]).contiguous()
        dres = dpre.reshape(-1, ctx.shape[-1]).contiguous() if dpre is not None else None
        if _use_native(dy2):
            from nanotron_b200.ops import native

            dx, dw, db = native.layernorm_bwd(dy2, pre, weight, mean, rstd, dres, ctx.has_bias)
        else:
            dx, dw, db = ref.layer_norm_bwd(dy2, pre, weight, mean, rstd, dres, ctx.has_bias)
        dx = dx.view(ctx.shape)
        return dx, dw.to(weight.dtype), (db.to(weight.dtype) if ctx.has_bias else None), None, (dx if ctx.has_residual else None)


def layer_norm(x, weight, bias, eps: float, residual=None):
    y, pre = _LayerNorm.apply(x, weight, bias, eps, residual)
    return y if residual is None else (y, pre)


# ============================================================================ rotary
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved, inplace, positions):
        ctx.save_for_backward(cos, sin, positions)
        ctx.interleaved = interleaved
        if _use_native(x):
            from nanotron_b200.ops import native

            out = native.rope(x, cos, sin, interleaved, inverse=False, inplace=inplace, positions=positions)
            if inplace:
                ctx.mark_dirty(x)
            return out
        if positions is not None:
            cos, sin = cos.index_select(0, positions.long()), sin.index_select(0, positions.long())
        return ref.rope_apply(x, cos, sin, interleaved)

    @staticmethod
    def backward(ctx, dout):
        cos, sin, positions = ctx.saved_tensors
        if _use_native(dout):
            from nanotron_b200.ops import native

            d = dout if dout.stride(-1) == 1 and dout.stride(0) % 8 == 0 and dout.stride(1) % 8 == 0 else dout.contiguous()
            return native.rope(d, cos, sin, ctx.interleaved, inverse=True, inplace=False, positions=positions), None, None, None, None, None
        if positions is not None:
            cos, sin = cos.index_select(0, positions.long()), sin.index_select(0, positions.long())
        return ref.rope_apply(dout, cos, sin, ctx.interleaved, inverse=True), None, None, None, None, None


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = False, inplace: bool = False, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x: [T, H, D] (may be a strided view into a fused qkv buffer, last dim contiguous).  cos/sin fp32: either
    per-token rows [T, D/2], or whole tables [P, D/2] indexed by ``positions`` [T] inside the kernel.
    The kernel wants head dims that are multiples of 16 and 16-byte aligned rows; other shapes (toy models) take the PyTorch
    composition, which autograd differentiates."""
    if x.is_cuda and _MODE != "torch" and not _rope_kernel_ok(x):
        if positions is not None:
            cos, sin = cos.index_select(0, positions.long()), sin.index_select(0, positions.long())
        return ref.rope_apply(x, cos, sin, interleaved)
    return _Rope.apply(x, cos, sin, interleaved, inplace, positions)


def _rope_kernel_ok(x: torch.Tensor) -> bool:
    return (x.dim() == 3 and x.shape[-1] % 16 == 0 and x.stride(-1) == 1 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
            and x.data_ptr() % 16 == 0 and x.dtype in (torch.bfloat16, torch.float16, torch.float32))


# ============================================================================ SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        if _use_native(gate_up):
            from nanotron_b200.ops import native

            return native.swiglu_fwd(gate_up.contiguous())
        return ref.swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, dout):
        (gate_up,) = ctx.saved_tensors
        if _use_native(dout):
            from nanotron_b200.ops import native

            return native.swiglu_bwd(gate_up.contiguous(), dout.contiguous())
        return ref.swiglu_bwd(gate_up, dout)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for the fused [gate | up] projection output; the product is recomputed in backward."""
    return _SwiGLU.apply(gate_up)


# ============================================================================ cross entropy pieces
def ce_partials(logits2: torch.Tensor, target: torch.Tensor, vocab_start: int):
    if _use_native(logits2):
        from nanotron_b200.ops import native

        return native.ce_partials(logits2.contiguous(), target.contiguous(), vocab_start)
    return ref.ce_partials(logits2, target, vocab_start)


def ce_backward(logits2, target, logz, grad_loss, grad_z, vocab_start: int):
    if _use_native(logits2):
        from nanotron_b200.ops import native

        return native.ce_backward(logits2, target, logz.contiguous(), grad_loss, grad_z, vocab_start)
    return ref.ce_backward(logits2, target, logz, grad_loss, grad_z, vocab_start)


# ============================================================================ attention
class _FlashAttnVarlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, window):
        from nanotron_b200.ops import native

        out, lse = native.flash_attn_fwd(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, window)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.cfg = (max_q, max_k, causal, scale, window)
        return out

    @staticmethod
    def backward(ctx, dout):
        from nanotron_b200.ops import native

        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, causal, scale, window = ctx.cfg
        dq, dk, dv = native.flash_attn_bwd(dout.contiguous(), q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal, scale, window)
        return dq, dk, dv, None, None, None, None, None, None, None


_WARNED = set()


def _warn_once(msg: str):
    if msg not in _WARNED:
        _WARNED.add(msg)
        import warnings

        warnings.warn(msg, stacklevel=3)


def _band_mask(lq: int, lk: int, causal: bool, window: Optional[int], device) -> Optional[torch.Tensor]:
    """Boolean [lq, lk] mask (True = attend) with the causal diagonal aligned to the bottom-right corner: query i sees keys
    j <= i + (lk - lq), and with a window only the last ``window`` of them, itself included (the convention of
    ``reference.attention_varlen`` and of the in-tree kernels)."""
    window = window if window else None
    if not causal and window is None:
        return None
    qi = torch.arange(lq, device=device).unsqueeze(1) + (lk - lq)
    kj = torch.arange(lk, device=device).unsqueeze(0)
    m = torch.ones(lq, lk, dtype=torch.bool, device=device)
    if causal:
        m &= kj <= qi
    if window is not None:
        m &= kj > qi - window
    return m


def _sdpa_varlen(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, window):
    """Library attention for CUDA tensors: the comparison path (``set_attention("sdpa")``) and shapes outside the in-tree kernel's
    contract (head dims other than 128, dtypes other than bf16).  Equal-length square causal batches take the library's own
    causal kernel; every other case (queries shorter than keys, windows, packed documents) runs the library kernel per
    document with an explicit bottom-right aligned mask, so the result always matches ``reference.attention_varlen``."""
    B = cu_q.numel() - 1
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    sdpa = torch.nn.functional.scaled_dot_product_attention
    if B * max_q == Tq and B * max_k == k.shape[0]:
        # equal-length rows (what a non-packed batch gives): no host read of cu_seqlens needed
        qb = q.view(B, max_q, Hq, D).transpose(1, 2)
        kb = k.view(B, max_k, Hkv, D).transpose(1, 2)
        vb = v.view(B, max_k, Hkv, D).transpose(1, 2)
        if window is None and (not causal or max_q == max_k):
            o = sdpa(qb, kb, vb, is_causal=causal, scale=scale, enable_gqa=Hq != Hkv)
        else:
            o = sdpa(qb, kb, vb, attn_mask=_band_mask(max_q, max_k, causal, window, q.device), scale=scale, enable_gqa=Hq != Hkv)
        return o.transpose(1, 2).reshape(Tq, Hq, D)
    _warn_once("ragged documents outside the in-tree attention kernel's contract: running the library kernel once per document")
    cq, ck = cu_q.tolist(), cu_k.tolist()
    outs = []
    for b in range(B):
        qd = q[cq[b] : cq[b + 1]].transpose(0, 1).unsqueeze(0)
        kd = k[ck[b] : ck[b + 1]].transpose(0, 1).unsqueeze(0)
        vd = v[ck[b] : ck[b + 1]].transpose(0, 1).unsqueeze(0)
        lq, lk = qd.shape[2], kd.shape[2]
        if lq == 0:
            continue
        if lk == 0:
            outs.append(torch.zeros(lq, Hq, D, dtype=q.dtype, device=q.device))
            continue
        o = sdpa(qd, kd, vd, attn_mask=_band_mask(lq, lk, causal, window, q.device), scale=scale, enable_gqa=Hq != Hkv)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, dim=0)


def flash_attn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, causal: bool = True, softmax_scale: Optional[float] = None, window: Optional[int] = None) -> torch.Tensor:
    """Variable-length attention over packed sequences.  q: [Tq,Hq,D]; k,v: [Tk,Hkv,D]; cu_seqlens int32 [B+1].
    Causal masks are aligned to the bottom-right corner when a sequence has fewer queries than keys.

    On CUDA the in-tree tcgen05 kernels run whenever their contract holds (bf16, head dim 128): packed documents, sliding windows
    and ``lq != lk`` included.  ``set_attention("sdpa")`` selects the library kernel for comparison runs; shapes outside the
    contract (toy head dims, fp32) also use it, with an explicit mask where one is needed.  The fp32 PyTorch oracle only runs
    on CPU tensors or under ``set_mode("torch")``."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and _MODE != "torch":
        from nanotron_b200.ops import native

        if _ATTN != "sdpa" and native.flash_attn_supported(q, k, v, window):
            return _FlashAttnVarlen.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, scale, window)
        return _sdpa_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, scale, window)
    return ref.attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=causal, softmax_scale=softmax_scale, window=window)


def attention_lse(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, causal: bool = True, softmax_scale: Optional[float] = None, window: Optional[int] = None) -> torch.Tensor:
    """log-sum-exp of the (scaled, masked) attention scores of every query: fp32 [Hq, Tq], no gradient.  A diagnostic (how
    peaked each head's softmax is; what the reference logs under the name ``attn_probs``, src/nanotron/models/qwen.py:309-328):
    it runs one extra attention forward."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    with torch.no_grad():
        if q.is_cuda and _MODE != "torch":
            from nanotron_b200.ops import native

            if native.flash_attn_supported(q, k, v, window):
                return native.flash_attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, scale, window)[1]
        return ref.attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=causal, softmax_scale=softmax_scale, window=window, return_lse=True)[1].float()


class _FusedQKVAttention(torch.autograd.Function):
    """RoPE (in place on the q / k parts of the fused projection output) + flash attention, with ONE gradient tensor for the
    whole qkv buffer: the attention backward writes dq / dk / dv into a single [T, (Hq + 2 Hkv) * D] buffer and the inverse
    rotation is applied in place, so autograd never materialises per-slice gradients or concatenates them."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, n_heads, n_kv, head_dim, cu, max_len, causal, scale, window, interleaved, use_rope):
        from nanotron_b200.ops import native

        T = qkv.shape[0]
        q = qkv[:, : n_heads * head_dim].view(T, n_heads, head_dim)
        k = qkv[:, n_heads * head_dim : (n_heads + n_kv) * head_dim].view(T, n_kv, head_dim)
        v = qkv[:, (n_heads + n_kv) * head_dim :].view(T, n_kv, head_dim)
        if use_rope:
            native.rope(q, cos, sin, interleaved, inverse=False, inplace=True, positions=positions)
            native.rope(k, cos, sin, interleaved, inverse=False, inplace=True, positions=positions)
        out, lse = native.flash_attn_fwd(q, k, v, cu, cu, max_len, max_len, causal, scale, window)
        ctx.save_for_backward(qkv, out, lse, cu, cos, sin, positions)
        ctx.cfg = (n_heads, n_kv, head_dim, max_len, causal, scale, window, interleaved, use_rope)
        return out

    @staticmethod
    def backward(ctx, dout):
        from nanotron_b200.ops import native

        qkv, out, lse, cu, cos, sin, positions = ctx.saved_tensors
        n_heads, n_kv, head_dim, max_len, causal, scale, window, interleaved, use_rope = ctx.cfg
        T = qkv.shape[0]
        q = qkv[:, : n_heads * head_dim].view(T, n_heads, head_dim)
        k = qkv[:, n_heads * head_dim : (n_heads + n_kv) * head_dim].view(T, n_kv, head_dim)
        v = qkv[:, (n_heads + n_kv) * head_dim :].view(T, n_kv, head_dim)
        dq, dk, dv = native.flash_attn_bwd(dout.contiguous(), q, k, v, out, lse, cu, cu, max_len, max_len, causal, scale, window)
        if use_rope:
            native.rope(dq, cos, sin, interleaved, inverse=True, inplace=True, positions=positions)
            native.rope(dk, cos, sin, interleaved, inverse=True, inplace=True, positions=positions)
        # dq is a view at offset 0 of the fused [T, Hq + 2 Hkv, D] gradient buffer
        dqkv = torch.as_strided(dq, (T, (n_heads + 2 * n_kv) * head_dim), ((n_heads + 2 * n_kv) * head_dim, 1), storage_offset=dq.storage_offset())
        return (dqkv,) + (None,) * 13


class _FusedQKVAttentionLib(torch.autograd.Function):
    """The same fusion around the LIBRARY attention kernel (equal-length causal sequences): RoPE in place on the q / k parts of
    the projection output, attention on the strided views, and a backward that rotates dq / dk straight into their slices of one
    [T, (Hq + 2 Hkv) * D] gradient buffer.  Without it autograd builds that buffer per layer from three zero fills, three
    strided copies and two full-size adds (the backward of slicing q, k and v out of qkv)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, n_heads, n_kv, head_dim, batch, seqlen, scale, interleaved, use_rope):
        from nanotron_b200.ops import native

        T = qkv.shape[0]
        q = qkv[:, : n_heads * head_dim].view(T, n_heads, head_dim)
        k = qkv[:, n_heads * head_dim : (n_heads + n_kv) * head_dim].view(T, n_kv, head_dim)
        v = qkv[:, (n_heads + n_kv) * head_dim :].view(T, n_kv, head_dim)
        if use_rope:
            native.rope(q, cos, sin, interleaved, inverse=False, inplace=True, positions=positions)
            native.rope(k, cos, sin, interleaved, inverse=False, inplace=True, positions=positions)
        needs_grad = ctx.needs_input_grad[0]
        with torch.set_grad_enabled(needs_grad):
            ql, kl, vl = (t.detach().requires_grad_(needs_grad) for t in (q, k, v))
            qb = ql.view(batch, seqlen, n_heads, head_dim).transpose(1, 2)
            kb = kl.view(batch, seqlen, n_kv, head_dim).transpose(1, 2)
            vb = vl.view(batch, seqlen, n_kv, head_dim).transpose(1, 2)
            o = torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, is_causal=True, scale=scale, enable_gqa=n_heads != n_kv)
            out = o.transpose(1, 2).reshape(T, n_heads, head_dim)
        ctx.inner = (ql, kl, vl, out) if needs_grad else None  # the library op's own graph: its backward is replayed below
        ctx.save_for_backward(cos, sin, positions)
        ctx.cfg = (n_heads, n_kv, head_dim, interleaved, use_rope, qkv.dtype)
        return out.detach()

    @staticmethod
    def backward(ctx, dout):
        from nanotron_b200.ops import native

        cos, sin, positions = ctx.saved_tensors
        n_heads, n_kv, head_dim, interleaved, use_rope, dtype = ctx.cfg
        ql, kl, vl, out = ctx.inner
        ctx.inner = None
        dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), dout)
        T = dq.shape[0]
        dqkv = torch.empty((T, (n_heads + 2 * n_kv) * head_dim), dtype=dtype, device=dq.device)
        gq = dqkv[:, : n_heads * head_dim].view(T, n_heads, head_dim)
        gk = dqkv[:, n_heads * head_dim : (n_heads + n_kv) * head_dim].view(T, n_kv, head_dim)
        gv = dqkv[:, (n_heads + n_kv) * head_dim :].view(T, n_kv, head_dim)
        if use_rope:
            dq = dq if dq.stride(-1) == 1 and dq.stride(0) % 8 == 0 and dq.stride(1) % 8 == 0 else dq.contiguous()
            dk = dk if dk.stride(-1) == 1 and dk.stride(0) % 8 == 0 and dk.stride(1) % 8 == 0 else dk.contiguous()
            native.rope(dq, cos, sin, interleaved, inverse=True, inplace=False, positions=positions, out=gq)
            native.rope(dk, cos, sin, interleaved, inverse=True, inplace=False, positions=positions, out=gk)
        else:
            gq.copy_(dq)
            gk.copy_(dk)
        gv.copy_(dv)
        return (dqkv,) + (None,) * 11


def fused_qkv_attention_supported(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window) -> bool:
    if not (qkv.is_cuda and _MODE != "torch" and _ATTN != "sdpa" and qkv.dtype == torch.bfloat16 and head_dim == 128 and qkv.is_contiguous()):
        return False
    from nanotron_b200.ops import native, native_attn

    native.lib()
    return native_attn._HAS["fwd"] and native_attn._HAS["bwd"] and n_heads % n_kv == 0


def fused_qkv_attention(qkv, cos_table, sin_table, positions, n_heads, n_kv, head_dim, cu_seqlens, max_seqlen, causal=True, softmax_scale=None, window=None, interleaved=False, use_rope=True):
    """qkv: [T, (Hq + 2 Hkv) * D] fresh output of the fused projection (it is rotated in place).  Returns [T, Hq, D]."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
    pos = positions.to(torch.int64).contiguous() if positions is not None else None
    return _FusedQKVAttention.apply(qkv, cos_table, sin_table, pos, n_heads, n_kv, head_dim, cu_seqlens.to(torch.int32), max_seqlen, causal, scale, window, interleaved, use_rope)


def fused_qkv_library_attention_supported(qkv: torch.Tensor, head_dim: int, window, cu_seqlens) -> bool:
    """Equal-length causal sequences (no packed documents, no window) on CUDA in bf16 / fp16 with the native element-wise kernels."""
    return (_use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float16) and qkv.is_contiguous() and head_dim % 16 == 0
            and qkv.data_ptr() % 16 == 0 and window is None and cu_seqlens is None)


def fused_qkv_library_attention(qkv, cos_table, sin_table, positions, n_heads, n_kv, head_dim, batch, seqlen, softmax_scale=None, interleaved=False, use_rope=True):
    """qkv: [batch * seqlen, (Hq + 2 Hkv) * D] fresh output of the fused projection (it is rotated in place).  Returns [T, Hq, D]."""
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
    pos = positions.to(torch.int64).contiguous() if positions is not None else None
    return _FusedQKVAttentionLib.apply(qkv, cos_table, sin_table, pos, n_heads, n_kv, head_dim, batch, seqlen, scale, interleaved, use_rope)


from nanotron_b200.ops import tp_fused  # noqa: E402,F401
