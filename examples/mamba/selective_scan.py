"""The selective state-space scan of Mamba in plain PyTorch (capability parity: reference examples/mamba/selective_scan_interface.py,
which wraps the ``mamba_ssm`` CUDA extension; that package and ``causal_conv1d`` are not installable here, so the example carries
its own scan).

    h_t = exp(dt_t * A) * h_{t-1} + dt_t * B_t * x_t          (state [d_inner, d_state] per sequence)
    y_t = <C_t, h_t> + D * x_t                                 out = y * silu(z)

``selective_scan_sequential`` is the literal recurrence (the oracle).  ``selective_scan`` works on chunks of ``chunk`` steps:
inside a chunk the decay between steps s <= t is exp(S_t - S_s) with S the running sum of dt * A, a lower-triangular matrix
whose entries never exceed 1 (no overflow however large dt gets), and the state is carried from chunk to chunk.  Both are
differentiable through autograd.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _prepare(u, delta, A, B, C, D, z, delta_bias, delta_softplus):
    dtype = u.dtype
    acc = torch.float64 if dtype == torch.float64 else torch.float32  # the recurrence runs in fp32 whatever the activations are
    u, delta = u.to(acc), delta.to(acc)
    if delta_bias is not None:
        delta = delta + delta_bias.to(acc)[None, :, None]
    if delta_softplus:
        delta = F.softplus(delta)
    return dtype, u, delta, A.to(acc), B.to(acc), C.to(acc), (D.to(acc) if D is not None else None), (z.to(acc) if z is not None else None)


def _finish(y, u, D, z, dtype):
    if D is not None:
        y = y + u * D[None, :, None]
    if z is not None:
        y = y * F.silu(z)
    return y.to(dtype)


def selective_scan_sequential(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, initial_state: Optional[torch.Tensor] = None, return_last_state: bool = False):
    """u, delta, z: [b, d, l]; A: [d, n]; B, C: [b, n, l]; D, delta_bias: [d].  Returns y [b, d, l] (and the last state [b, d, n])."""
    dtype, u, delta, A, B, C, D, z = _prepare(u, delta, A, B, C, D, z, delta_bias, delta_softplus)
    b, d, l = u.shape
    h = initial_state.to(u.dtype) if initial_state is not None else u.new_zeros(b, d, A.shape[1])
    ys = []
    for t in range(l):
        decay = torch.exp(delta[:, :, t, None] * A[None])  # [b, d, n]
        h = decay * h + delta[:, :, t, None] * B[:, None, :, t] * u[:, :, t, None]
        ys.append(torch.einsum("bdn,bn->bd", h, C[:, :, t]))
    y = _finish(torch.stack(ys, dim=2), u, D, z, dtype)
    return (y, h) if return_last_state else y


def selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, chunk: int = 32, initial_state: Optional[torch.Tensor] = None, return_last_state: bool = False):
    """Same contract as ``selective_scan_sequential``; ``chunk`` steps are handled at once."""
    dtype, u, delta, A, B, C, D, z = _prepare(u, delta, A, B, C, D, z, delta_bias, delta_softplus)
    b, d, l = u.shape
    n = A.shape[1]
    h = initial_state.to(u.dtype) if initial_state is not None else u.new_zeros(b, d, n)
    outs = []
    for start in range(0, l, chunk):
        sl = slice(start, min(l, start + chunk))
        dt, uc, Bc, Cc = delta[:, :, sl], u[:, :, sl], B[:, :, sl], C[:, :, sl]
        T = dt.shape[2]
        S = torch.cumsum(dt[..., None] * A[None, :, None, :], dim=2)  # [b, d, T, n], non-increasing along T
        inp = dt[..., None] * Bc.transpose(1, 2)[:, None] * uc[..., None]  # [b, d, T, n]: what step s adds to the state
        # W[t, s] = exp(S_t - S_s) for s <= t, else 0
        diff = S[:, :, :, None, :] - S[:, :, None, :, :]  # [b, d, T(t), T(s), n]
        keep = torch.ones(T, T, dtype=torch.bool, device=u.device).tril()[None, None, :, :, None]
        W = torch.where(keep, torch.exp(torch.where(keep, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
        states = torch.einsum("bdtsn,bdsn->bdtn", W, inp) + torch.exp(S) * h[:, :, None, :]
        outs.append(torch.einsum("bdtn,bnt->bdt", states, Cc))
        h = states[:, :, -1]
    y = _finish(torch.cat(outs, dim=2), u, D, z, dtype)
    return (y, h) if return_last_state else y


def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decoding step.  state: [b, d, n]; x, dt, z: [b, d]; B, C: [b, n].  Returns (y [b, d], new state)."""
    dt = dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    if dt_softplus:
        dt = F.softplus(dt)
    new = torch.exp(dt[..., None] * A.float()[None]) * state.float() + dt[..., None] * B.float()[:, None, :] * x.float()[..., None]
    y = torch.einsum("bdn,bn->bd", new, C.float())
    if D is not None:
        y = y + D.float() * x.float()
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(x.dtype), new
