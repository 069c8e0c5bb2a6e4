"""Bindings of the tcgen05 GEMM kernels (``csrc/gemm_tcgen05.cu``)."""
from __future__ import annotations

import torch

_HAS = {"gemm": False}


def declare(L):
    _HAS["gemm"] = hasattr(L, "ntb_gemm_bf16")


def gemm_supported(a: torch.Tensor, b: torch.Tensor, force: bool = False) -> bool:
    return False


def gemm_nt(a, b):
    raise NotImplementedError


def gemm_nn(a, b):
    raise NotImplementedError


def gemm_tn(a, b):
    raise NotImplementedError


def gemm_tn_accum_fp32(a, b, out):
    raise NotImplementedError
