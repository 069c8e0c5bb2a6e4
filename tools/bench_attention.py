"""Flash attention micro-benchmark: in-tree tcgen05 forward vs the library (SDPA) forward on Llama-3-8B shapes.

    python tools/bench_attention.py
FLOPs are counted for the causal half (2 * 2 * H * S^2 * D / 2 per sequence).
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import math

import torch

from bench_kernels import _peaks, time_fn


def main():
    from nanotron_b200.ops import native, native_attn, native_gemm

    native.lib()
    peak = _peaks()["bf16_tflops"]
    for (B, S, Hq, Hkv) in [(1, 4096, 32, 8), (2, 4096, 32, 8), (1, 8192, 32, 8), (1, 16384, 32, 8)]:
        T = B * S
        qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
        q = qkv[:, : Hq * 128].view(T, Hq, 128)
        k = qkv[:, Hq * 128 : (Hq + Hkv) * 128].view(T, Hkv, 128)
        v = qkv[:, (Hq + Hkv) * 128 :].view(T, Hkv, 128)
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
        scale = 1 / math.sqrt(128)
        flops = 4.0 * B * Hq * S * S * 128 / 2
        native_attn.set_forward_variant("one_tile")
        ms1 = time_fn(lambda: native_attn.flash_attn_fwd(q, k, v, cu, cu, S, S, True, scale, None))
        native_attn.set_forward_variant("two_tile")
        ms = time_fn(lambda: native_attn.flash_attn_fwd(q, k, v, cu, cu, S, S, True, scale, None))
        native_gemm.check_status("cuda")
        qb = q.reshape(B, S, Hq, 128).transpose(1, 2)
        kb = k.reshape(B, S, Hkv, 128).transpose(1, 2)
        vb = v.reshape(B, S, Hkv, 128).transpose(1, 2)
        ms_lib = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, is_causal=True, enable_gqa=True))
        # backward (in-tree) vs library backward
        out, lse = native_attn.flash_attn_fwd(q, k, v, cu, cu, S, S, True, scale, None)
        dout = torch.randn_like(out)
        ms_b = time_fn(lambda: native_attn.flash_attn_bwd(dout, q, k, v, out, lse, cu, cu, S, S, True, scale, None))
        native_gemm.check_status("cuda")
        qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (qb, kb, vb))
        o = torch.nn.functional.scaled_dot_product_attention(qg, kg, vg, is_causal=True, enable_gqa=True)
        go = torch.randn_like(o)
        ms_lb = time_fn(lambda: torch.autograd.grad(o, (qg, kg, vg), go, retain_graph=True))
        print(f"B={B} S={S} bwd: tcgen05 {ms_b:7.3f} ms {2.5 * flops / ms_b / 1e9:7.1f} TFLOP/s | library {ms_lb:7.3f} ms {2.5 * flops / ms_lb / 1e9:7.1f} TFLOP/s", flush=True)
        print(f"B={B} S={S} Hq={Hq} Hkv={Hkv}  tcgen05 fwd, one query tile per CTA {ms1:7.3f} ms {flops / ms1 / 1e9:7.1f} TFLOP/s", flush=True)
        print(f"B={B} S={S} Hq={Hq} Hkv={Hkv}  tcgen05 fwd {ms:7.3f} ms {flops / ms / 1e9:7.1f} TFLOP/s ({flops / ms / 1e9 / peak:4.2f} of measured GEMM peak) | library fwd {ms_lib:7.3f} ms {flops / ms_lib / 1e9:7.1f} TFLOP/s", flush=True)


if __name__ == "__main__":
    main()
