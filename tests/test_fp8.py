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
