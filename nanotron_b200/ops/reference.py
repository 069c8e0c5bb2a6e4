"""Plain PyTorch fp32 implementations of every hot op.

These are the numerical oracles for the CUDA kernels and the implementation used on CPU.  They are written for
clarity, not speed: statistics in fp32, outputs cast back to the input dtype.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ norms
def rms_norm_fwd(x, weight, eps: float, residual=None):
    """Returns (y, pre_norm, rstd).  pre_norm = x + residual (the new residual stream), in x.dtype."""
    pre = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    pf = pre.float()
    rstd = torch.rsqrt(pf.pow(2).mean(-1, keepdim=True) + eps)
    y = (pf * rstd * weight.float()).to(x.dtype)
    return y, pre, rstd.squeeze(-1)


def rms_norm_bwd(dy, pre, weight, rstd, dresidual=None):
    """Returns (dx, dweight[fp32]).  dx also flows to the residual input (same tensor)."""
    pf, dyf, wf = pre.float(), dy.float(), weight.float()
    xhat = pf * rstd.unsqueeze(-1)
    dw = (dyf * xhat).reshape(-1, pf.shape[-1]).sum(0)
    wdy = dyf * wf
    c1 = (wdy * xhat).mean(-1, keepdim=True)
    dx = (wdy - xhat * c1) * rstd.unsqueeze(-1)
    if dresidual is not None:
        dx = dx + dresidual.float()
    return dx.to(pre.dtype), dw


def layer_norm_fwd(x, weight, bias, eps: float, residual=None):
    pre = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    pf = pre.float()
    mean = pf.mean(-1, keepdim=True)
    var = (pf - mean).pow(2).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (pf - mean) * rstd * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype), pre, mean.squeeze(-1), rstd.squeeze(-1)


def layer_norm_bwd(dy, pre, weight, mean, rstd, dresidual=None, has_bias=True):
    pf, dyf, wf = pre.float(), dy.float(), weight.float()
    xhat = (pf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
    dw = (dyf * xhat).reshape(-1, pf.shape[-1]).sum(0)
    db = dyf.reshape(-1, pf.shape[-1]).sum(0) if has_bias else None
    wdy = dyf * wf
    c1 = (wdy * xhat).mean(-1, keepdim=True)
    c2 = wdy.mean(-1, keepdim=True)
    dx = (wdy - xhat * c1 - c2) * rstd.unsqueeze(-1)
    if dresidual is not None:
        dx = dx + dresidual.float()
    return dx.to(pre.dtype), dw, db


# ------------------------------------------------------------------ rotary
def rope_inverse_frequencies(dim: int, theta: float, scaling: Optional[dict] = None, device=None) -> torch.Tensor:
    """The dim/2 rotation frequencies, with the ``rope_scaling`` rules of Hugging Face model configurations applied:

    * ``linear``: every frequency divided by ``factor`` (position interpolation);
    * ``llama3``: wavelengths longer than ``original_max_position_embeddings / low_freq_factor`` are stretched by ``factor``,
      those shorter than ``original / high_freq_factor`` are kept, the band in between is blended linearly (Llama-3.1).

    Other rules (``dynamic``, ``yarn``, ``longrope``) are not implemented and raise instead of training with silently different
    positions.  (The reference carries ``rope_scaling`` in its configurations but never reads it.)"""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    if not scaling:
        return inv_freq
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in (None, "default"):
        return inv_freq
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind == "llama3":
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv_freq
        blend = ((original / wavelen - low) / (high - low)).clamp(0.0, 1.0)  # 0: long wavelengths (stretched), 1: short ones (kept)
        return (1 - blend) * inv_freq / factor + blend * inv_freq
    raise NotImplementedError(f"rope_scaling of type {kind!r} is not implemented (supported: linear, llama3)")


def rope_cos_sin(positions: torch.Tensor, dim: int, theta: float, interpolation_factor: Optional[float] = None, dtype=torch.float32, scaling: Optional[dict] = None):
    """cos/sin tables [*positions.shape, dim/2] in fp32."""
    inv_freq = rope_inverse_frequencies(dim, theta, scaling, device=positions.device)
    pos = positions.float()
    if interpolation_factor is not None:
        pos = pos / interpolation_factor
    ang = pos.unsqueeze(-1) * inv_freq
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = False, inverse: bool = False):
    """x: [T, H, D]; cos/sin: [T, D/2].  Non-interleaved rotates (x[..., :D/2], x[..., D/2:]) pairs (HF / Llama-3
    layout); interleaved rotates (x[..., 0::2], x[..., 1::2]).  ``inverse`` applies the transposed rotation (backward)."""
    xf = x.float()
    c = cos.float().unsqueeze(-2)
    s = sin.float().unsqueeze(-2)
    if inverse:
        s = -s
    if interleaved:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        x1, x2 = xf[..., :h], xf[..., h:]
        o = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)
    return o.to(x.dtype)


# ------------------------------------------------------------------ activations
def swiglu_fwd(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up: [..., 2*I] laid out as [gate | up]; returns silu(gate) * up."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def swiglu_bwd(gate_up: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    d = dout.float()
    sig = torch.sigmoid(g)
    dg = d * u * sig * (1 + g * (1 - sig))
    du = d * g * sig
    return torch.cat([dg, du], dim=-1).to(gate_up.dtype)


# ------------------------------------------------------------------ cross entropy
def ce_partials(logits: torch.Tensor, target: torch.Tensor, vocab_start: int):
    """Per-row (max, sum exp(l - max), target logit or 0 when the target is outside this shard), all fp32."""
    lf = logits.float()
    m = lf.max(dim=-1).values
    s = torch.exp(lf - m.unsqueeze(-1)).sum(-1)
    local = target - vocab_start
    inside = (local >= 0) & (local < logits.shape[-1])
    idx = local.clamp(0, logits.shape[-1] - 1)
    t = lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1)
    t = torch.where(inside, t, torch.zeros_like(t))
    return m, s, t


def ce_backward(logits, target, logz, grad_loss, grad_z, vocab_start: int):
    """d logits = (g + gz) * softmax - g * onehot, in logits.dtype."""
    lf = logits.float()
    p = torch.exp(lf - logz.unsqueeze(-1))
    coef = grad_loss if grad_z is None else grad_loss + grad_z
    g = p * coef.unsqueeze(-1)
    local = target - vocab_start
    inside = (local >= 0) & (local < logits.shape[-1])
    idx = local.clamp(0, logits.shape[-1] - 1)
    sub = torch.where(inside, grad_loss, torch.zeros_like(grad_loss))
    g.scatter_add_(-1, idx.unsqueeze(-1), -sub.unsqueeze(-1))
    return g.to(logits.dtype)


# ------------------------------------------------------------------ attention
def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal: bool = True, softmax_scale: Optional[float] = None, window: Optional[int] = None, return_lse: bool = False, q_offsets=None):
    """q: [Tq, Hq, D], k/v: [Tk, Hkv, D]; sequences delimited by cu_seqlens (int32 [B+1]).
    Causal alignment is bottom-right (query i of a sequence of length Lq sees keys <= i + Lk - Lq), the
    flash-attention convention.  ``q_offsets`` (int [B]) overrides that shift per sequence (used by context
    parallelism where the local queries sit at an arbitrary global position).  fp32 math."""
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros_like(q, dtype=torch.float32)
    lse = torch.full((Hq, Tq), float("-inf"), dtype=torch.float32, device=q.device)
    B = cu_seqlens_q.numel() - 1
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for b in range(B):
        qs, qe, ks, ke = cq[b], cq[b + 1], ck[b], ck[b + 1]
        lq, lk = qe - qs, ke - ks
        if lq == 0:
            continue
        qb = q[qs:qe].float().transpose(0, 1)  # [Hq, lq, D]
        kb = k[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vb = v[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qb, kb.transpose(1, 2)) * scale
        shift = (lk - lq) if q_offsets is None else int(q_offsets[b])
        qi = torch.arange(lq, device=q.device).unsqueeze(1) + shift
        ki = torch.arange(lk, device=q.device).unsqueeze(0)
        mask = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if causal:
            mask &= ki <= qi
        if window is not None and window > 0:
            mask &= ki > qi - window
        s = s.masked_fill(~mask, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)
        out[qs:qe] = torch.matmul(p, vb).transpose(0, 1)
        lse[:, qs:qe] = l
    o = out.to(q.dtype)
    return (o, lse) if return_lse else o


# ------------------------------------------------------------------ optimizer
def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """In-place AdamW on fp32 tensors; matches torch.optim.AdamW (decoupled decay, bias correction)."""
    g = g * grad_scale
    p.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
