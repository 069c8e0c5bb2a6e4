import pytest
import torch

from nanotron_b200.fp8 import FP8Linear, dequantize, quantize_1x128, quantize_128x128
from nanotron_b200.fp8.quantize import quantize_1x128_reference


def test_block_quantisation_round_trip_error_is_bounded():
    torch.manual_seed(0)
    x = torch.randn(37, 300) * torch.logspace(-3, 3, 300)  # wide dynamic range across columns
    for q, fn in ((torch.float8_e4m3fn, quantize_1x128), (torch.float8_e5m2, quantize_1x128)):
        t = fn(x, q)
        back = dequantize(t, torch.float32)
        rel = ((back - x).abs() / x.abs().clamp(min=1e-6))
        # inside a block everything is scaled by the block max: error relative to the block max is <= half an ulp
        blk_max = torch.nn.functional.pad(x.abs(), (0, 84)).view(37, -1, 128).amax(-1).repeat_interleave(128, 1)[:, :300]
        assert ((back - x).abs() <= blk_max * (0.07 if q == torch.float8_e4m3fn else 0.14)).all()
    w = torch.randn(200, 260)
    t = quantize_128x128(w)
    assert t.scale.shape == (2, 3)
    assert (dequantize(t, torch.float32) - w).abs().max() < 0.07 * w.abs().max()


def test_fp8_linear_trains_close_to_fp32():
    torch.manual_seed(1)
    lin = FP8Linear(256, 128, bias=True)
    ref = torch.nn.Linear(256, 128, bias=True)
    ref.load_state_dict(lin.state_dict())
    x = torch.randn(64, 256)
    y, y0 = lin(x), ref(x)
    assert (y - y0).abs().max() < 0.05 * y0.abs().max()
    g = torch.randn_like(y)
    y.backward(g)
    y0.backward(g)
    assert (lin.weight.grad - ref.weight.grad).abs().max() < 0.08 * ref.weight.grad.abs().max()


@pytest.mark.gpu
def test_fp8_quantize_kernel_matches_reference():
    torch.manual_seed(2)
    x = (torch.randn(129, 512, device="cuda") * 3).to(torch.bfloat16)
    for q in (torch.float8_e4m3fn, torch.float8_e5m2):
        got = quantize_1x128(x, q)
        exp = quantize_1x128_reference(x, q)
        torch.testing.assert_close(got.scale, exp.scale, rtol=1e-6, atol=0)
        torch.testing.assert_close(dequantize(got, torch.float32), dequantize(exp, torch.float32), rtol=0.13, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (384, 256, 1024), (130, 264, 208)])
def test_fp8_tensor_core_gemm_matches_dequantised_product(M, N, K):
    from nanotron_b200.fp8.quantize import dequantize, quantize_1x128_reference, quantize_128x128_reference
    from nanotron_b200.ops import native, native_gemm

    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    for a_dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        xq = quantize_1x128_reference(x, a_dtype)
        wq = quantize_128x128_reference(w, torch.float8_e4m3fn)
        exp = dequantize(xq, torch.float32) @ dequantize(wq, torch.float32).t()
        got = native.gemm_fp8_blockscaled(xq, wq)
        native_gemm.check_status("cuda")
        torch.testing.assert_close(got.float(), exp, atol=2e-2 * float(exp.abs().max()), rtol=2e-2)
        # both operands with per-row scales (the weight-gradient form), accumulated into fp32
        wq_row = quantize_1x128_reference(w, torch.float8_e4m3fn)
        exp_row = dequantize(xq, torch.float32) @ dequantize(wq_row, torch.float32).t()
        acc = torch.full((M, N), 0.5, device="cuda", dtype=torch.float32)
        native.gemm_fp8_blockscaled(xq, wq_row, out=acc, accumulate_fp32=True)
        native_gemm.check_status("cuda")
        torch.testing.assert_close(acc, exp_row + 0.5, atol=1e-3 * float(exp_row.abs().max()) + 1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_fp8_linear_native_path_matches_dequantised_path():
    from nanotron_b200 import ops
    from nanotron_b200.fp8.linear import FP8Linear

    torch.manual_seed(0)
    lin = FP8Linear(512, 384, bias=False).cuda().to(torch.bfloat16)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    res = {}
    for mode in ("auto", "torch"):
        ops.set_mode(mode)
        try:
            lin.weight.grad = None
            xi = x.clone().requires_grad_(True)
            y = lin(xi)
            y.backward(g)
            res[mode] = (y.detach().float(), xi.grad.float(), lin.weight.grad.float().clone())
        finally:
            ops.set_mode("auto")
    for a, b, name in zip(res["auto"], res["torch"], ("y", "dx", "dW")):
        err = (a - b).abs().max() / b.abs().max()
        assert err < 2e-2, (name, float(err))


def test_fp8_linear_mode_is_reachable_from_the_config_and_tracks_bf16():
    """``kernels.linear: fp8`` routes the three products of every tensor-parallel linear through block-scaled fp8 operands; the
    loss curve of a small model stays close to the full-precision one."""
    import nanotron_b200.config as c
    from helpers import make_config, single_process_env, tiny_llama_config
    from nanotron_b200 import ops
    from nanotron_b200.fp8 import linear as fp8_linear
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    def run(linear):
        single_process_env()
        cfg = make_config(tiny_llama_config(hidden_size=128, intermediate_size=256, num_attention_heads=2, num_key_value_heads=2, vocab_size=256), seq=64, mbs=2, steps=6, lr=3e-3)
        cfg.kernels = c.KernelArgs(linear=linear)
        t = T(cfg)
        t.prepare_training()
        g = torch.Generator().manual_seed(0)
        tokens = torch.randint(0, 256, (2, 65), generator=g)
        batch = {"input_ids": tokens[:, :-1].contiguous(), "input_mask": torch.ones(2, 64, dtype=torch.bool), "label_ids": tokens[:, 1:].contiguous(), "label_mask": torch.ones(2, 64, dtype=torch.bool)}
        losses = []
        for _ in range(6):
            _, loss, _ = t.training_step(iter([batch]))
            t.iteration_step += 1
            losses.append(float(loss))
        t.parallel_context.destroy()
        return losses

    calls = {"n": 0}
    orig = fp8_linear.fp8_forward

    def counting(x2, w):
        calls["n"] += 1
        return orig(x2, w)

    fp8_linear.fp8_forward = counting
    try:
        fp8 = run("fp8")
    finally:
        fp8_linear.fp8_forward = orig
        ops.set_linear("bf16")
    assert calls["n"] >= 6 * 2 * 4  # qkv, o, gate_up, down of both layers, every step
    ref = run("bf16")
    assert fp8[-1] < fp8[0] - 0.3, fp8
    for a, b in zip(fp8, ref):
        assert abs(a - b) < 0.05, (fp8, ref)


def test_weight_copies_are_quantised_once_per_weights_generation():
    """The e4m3 copy of a weight (and its transposed copy for the dgrad) is computed once and reused by every micro-batch until
    the weights change: an in-place update (autograd version) or an explicit new generation (optimizer kernels that write
    through raw pointers) makes the next use recompute it."""
    from nanotron_b200.fp8 import QuantizedWeightCache, dequantize
    from nanotron_b200.fp8 import linear as fp8_linear

    cache = QuantizedWeightCache()
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(256, 384))
    a = cache.get(w)
    assert cache.get(w) is a and (cache.hits, cache.misses) == (1, 1)
    t = cache.get(w, transposed=True)
    assert t.data.shape == (384, 256) and torch.equal(t.data.t().float(), a.data.float()) and torch.equal(t.scale.t(), a.scale)
    assert cache.get(w, transposed=True) is t
    with torch.no_grad():
        w.mul_(2.0)  # in-place update: the version counter moves
    b = cache.get(w)
    assert b is not a and torch.allclose(dequantize(b, torch.float32), 2 * dequantize(a, torch.float32), rtol=0, atol=1e-6)
    w.data.copy_(torch.randn(256, 384))  # a raw write that autograd does not see ...
    assert cache.get(w) is b  # ... is only caught by a new generation
    cache.invalidate()
    c = cache.get(w)
    assert c is not b and not torch.equal(c.data.float(), b.data.float())
    # the linear layer goes through the shared cache: several micro-batches, one quantisation; numerics unchanged
    shared = fp8_linear.weight_cache
    shared.invalidate()
    h0, m0 = shared.hits, shared.misses
    lin = torch.nn.Linear(384, 256, bias=False)
    x = torch.randn(128, 384)
    outs = [fp8_linear.fp8_forward(x, lin.weight) for _ in range(3)]
    assert shared.misses - m0 == 1 and shared.hits - h0 == 2 and all(torch.equal(o, outs[0]) for o in outs)
    shared.enabled = False
    try:
        assert torch.equal(fp8_linear.fp8_forward(x, lin.weight), outs[0])
    finally:
        shared.enabled = True


def test_per_tensor_power_of_two_scaling_round_trips():
    from nanotron_b200.fp8 import DTypes, FP8Tensor, convert_tensor_from_fp8
    from nanotron_b200.fp8.tensor import compute_scale
    from nanotron_b200.fp8.utils import is_overflow_underflow_nan, quantization_error

    torch.manual_seed(1)
    x = torch.randn(64, 64) * 3.0
    for dtype, tol in ((DTypes.FP8E4M3, 0.07), (DTypes.FP8E5M2, 0.13)):
        q = FP8Tensor(x, dtype)
        scale = float(q.fp8_meta.scale)
        assert scale == 2.0 ** round(torch.log2(torch.tensor(scale)).item())  # a power of two
        assert float(x.abs().max()) * scale <= q.fp8_meta.fp8_max < float(x.abs().max()) * scale * 2  # the largest that fits
        back = q.to_float()
        assert not is_overflow_underflow_nan(back) and quantization_error(x, back)["max_rel"] < tol
        assert torch.equal(back, convert_tensor_from_fp8(q.data, q.fp8_meta))
    assert float(compute_scale(torch.tensor(0.0), DTypes.FP8E4M3)) == 1.0
    q = FP8Tensor(x, DTypes.FP8E4M3)
    old = float(q.fp8_meta.scale)
    q.set_data(x * 1.1)  # still fits: the scale stays
    assert float(q.fp8_meta.scale) == old or float(x.abs().max()) * 1.1 * old > q.fp8_meta.fp8_max
    q.set_data(x * 64)  # would overflow: rescaled
    assert float(q.fp8_meta.scale) < old and not is_overflow_underflow_nan(q.to_float())


def test_cached_copy_dies_with_its_weight():
    """A weight that was freed may give its address to a new tensor of the same shape: the new tensor must not inherit the copy."""
    from nanotron_b200.fp8 import QuantizedWeightCache

    cache = QuantizedWeightCache()
    w = torch.randn(128, 128)
    first = cache.get(w)
    key_count = len(cache._entries)
    ptr = w.data_ptr()
    del w
    for _ in range(50):  # try to land on the same address
        v = torch.randn(128, 128)
        if v.data_ptr() == ptr:
            got = cache.get(v)
            assert got is not first and cache.misses == 2
            break
        del v
    assert len(cache._entries) >= key_count
    # an alias of a live weight (what autograd hands back in backward) does share the copy
    w2 = torch.nn.Parameter(torch.randn(128, 128))
    c = cache.get(w2)
    assert cache.get(w2.detach()) is c
