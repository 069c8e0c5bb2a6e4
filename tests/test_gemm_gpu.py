"""tcgen05 GEMM against an fp32 PyTorch product: every operand layout, every output mode, edge tiles."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=["single", "pair"], autouse=True)
def gemm_variant(request):
    """Every test runs on both in-tree kernels: one CTA per tile, and CTA pairs (cta_group::2)."""
    from nanotron_b200.ops import native_gemm

    old = native_gemm.VARIANT["kernel"]
    native_gemm.set_variant(request.param)
    yield request.param
    native_gemm.set_variant(old)


def _rel_err(got, exp):
    return ((got.float() - exp).abs().max() / exp.abs().max().clamp(min=1e-6)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (192, 320, 448), (1024, 1536, 1024), (4096, 6144, 4096)])
def test_gemm_nt(M, N, K):
    from nanotron_b200.ops import native_gemm as g
    from nanotron_b200.ops import native

    native.lib()
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    exp = x.float() @ w.float().t()
    got = g.gemm_nt(x, w)
    g.check_status(DEV)
    assert _rel_err(got, exp) < 1e-2
    got32 = g.gemm_nt(x, w, out_dtype=torch.float32)
    assert _rel_err(got32, exp) < 1e-3


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (320, 192, 448), (2048, 1024, 3072)])
def test_gemm_nn_and_tn(M, N, K):
    from nanotron_b200.ops import native_gemm as g
    from nanotron_b200.ops import native

    native.lib()
    torch.manual_seed(1)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    dx = g.gemm_nn(dy, w)
    assert _rel_err(dx, dy.float() @ w.float()) < 1e-2
    dw = g.gemm_tn(dy, x)
    exp_dw = dy.float().t() @ x.float()
    assert _rel_err(dw, exp_dw) < 1e-2
    acc = torch.randn(N, K, device=DEV, dtype=torch.float32)
    base = acc.clone()
    g.gemm_tn_accum_fp32(dy, x, acc)
    g.gemm_tn_accum_fp32(dy, x, acc)
    g.check_status(DEV)
    assert _rel_err(acc - base, 2 * exp_dw) < 1e-3


def test_linear_ops_route_to_tcgen05():
    from nanotron_b200 import ops

    ops.set_gemm("tcgen05")
    try:
        torch.manual_seed(2)
        x = torch.randn(512, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        lin = torch.nn.Linear(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16)
        n0 = ops.native_launches()
        y = ops.linear_forward(x, lin.weight)
        assert ops.native_launches() == n0 + 1
        exp = torch.nn.functional.linear(x.float(), lin.weight.float())
        assert _rel_err(y, exp) < 1e-2
    finally:
        ops.set_gemm("auto")


@pytest.mark.parametrize("M,N,K", [(1024, 2048, 1024), (4096, 1536, 4096), (512, 512, 4096), (512, 1024, 2368), (320, 448, 2048), (8192, 3584, 4096)])
def test_pair_kernel_splits_the_last_round_along_k(M, N, K, gemm_variant):
    """Tile counts that leave the last round of CTA pairs mostly idle: the pair kernel cuts those tiles along K (fp32 partial
    sums parked in workspace slabs, summed in chunk order by a fix-up pass).  Results must match the fp32 product and the
    unsplit launch, for every output mode, and be the same bits on every launch."""
    if gemm_variant != "pair":
        pytest.skip("only the pair kernel splits")
    from nanotron_b200.ops import native, native_gemm as g

    native.lib()
    torch.manual_seed(3)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    exp = x.float() @ w.float().t()
    whole = g.gemm_nt(x, w)  # the default: whole tiles
    g.set_split(True)
    try:
        _check_split_products(g, x, w, exp, whole, M, N, K)
    finally:
        g.set_split(False)


def _check_split_products(g, x, w, exp, whole, M, N, K):
    first = None
    for _ in range(3):
        got = g.gemm_nt(x, w)
        g.check_status(DEV)
        assert _rel_err(got, exp) < 1e-2
        assert _rel_err(got, whole.float()) < 1e-2
        first = got if first is None else first
        assert torch.equal(got, first)
    got32 = g.gemm_nt(x, w, out_dtype=torch.float32)
    assert _rel_err(got32, exp) < 1e-3
    # dgrad (B read MN-major), wgrad in bf16 and with fp32 accumulation
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    dx = g.gemm_nn(dy, w)
    assert _rel_err(dx, dy.float() @ w.float()) < 1e-2
    dw = g.gemm_tn(dy, x)
    exp_dw = dy.float().t() @ x.float()
    assert _rel_err(dw, exp_dw) < 1e-2
    acc = torch.randn(N, K, device=DEV, dtype=torch.float32)
    base = acc.clone()
    g.gemm_tn_accum_fp32(dy, x, acc)
    g.gemm_tn_accum_fp32(dy, x, acc)
    g.check_status(DEV)
    assert _rel_err(acc - base, 2 * exp_dw) < 1e-3
