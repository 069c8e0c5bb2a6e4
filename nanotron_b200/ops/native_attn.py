"""Bindings of the flash-attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

import torch

_HAS = {"attn": False}


def declare(L):
    _HAS["attn"] = hasattr(L, "ntb_flash_attn_fwd")


def flash_attn_supported(q, k, v, window) -> bool:
    return False


def flash_attn_fwd(*a, **k):
    raise NotImplementedError


def flash_attn_bwd(*a, **k):
    raise NotImplementedError
