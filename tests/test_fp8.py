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
