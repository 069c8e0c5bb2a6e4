"""Mixture-of-experts kernels on one GPU: the device-side plan / dispatch / combine against index arithmetic, the tcgen05
grouped GEMMs against per-expert fp32 matmuls, and the whole fused layer (forward + backward) against the PyTorch path."""
import pytest
import torch

from helpers import single_process_env, tiny_qwen_config

pytestmark = pytest.mark.gpu


def _routing(T, E, k, seed=0, empty_expert=None):
    g = torch.Generator(device="cuda").manual_seed(seed)
    scores = torch.rand(T, E, device="cuda", generator=g)
    if empty_expert is not None:
        scores[:, empty_expert] = -1.0
    top_p, top_i = torch.topk(torch.softmax(scores * 4, -1), k, dim=-1)
    counts = torch.bincount(top_i.reshape(-1), minlength=E).to(torch.int32)
    return top_p.float().contiguous(), top_i.to(torch.int32).contiguous(), counts


def test_plan_rank_dispatch_combine_roundtrip():
    from nanotron_b200.ops import moe_fused

    T, E, k, h = 300, 8, 2, 256
    top_p, top_i, counts = _routing(T, E, k, empty_expert=3)
    ctx = moe_fused.get_context(None, h, T, k, E)
    plan = ctx.make_plan(counts, top_i)
    torch.cuda.synchronize()
    ctx.check()
    seg = plan.seg_off.tolist()
    cnt = counts.tolist()
    assert seg[0] == 0 and all(s % 128 == 0 for s in seg)
    assert [seg[i + 1] - seg[i] for i in range(E)] == [((c + 127) // 128) * 128 for c in cnt]
    assert plan.cnt_tot.tolist() == cnt
    assert int(plan.num_m_tiles) == seg[-1] // 128
    te = plan.tile_expert.tolist()
    for e in range(E):
        assert all(te[i] == e for i in range(seg[e] // 128, seg[e + 1] // 128))
    # rows: token order inside each expert, every row used exactly once
    flat_e = top_i.reshape(-1)
    for e in range(E):
        assert plan.row_of[flat_e == e].tolist() == list(range(seg[e], seg[e] + cnt[e]))
    row_of = plan.row_of.view(T, k).cpu()
    x = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    ctx.recv.tensor.fill_(7.0)  # stale data: the padding must come out zero
    ctx.dispatch(x, top_i, plan, top_p, zero_pad=True)
    recv = ctx.recv.tensor.view(ctx.cap_rows, h)
    for t in (0, 17, T - 1):
        for j in range(k):
            assert torch.equal(recv[int(row_of[t, j])], x[t])
            assert float(ctx.p_recv.tensor[int(row_of[t, j])]) == float(top_p[t, j])
    for e in range(E):
        if seg[e + 1] > seg[e] + cnt[e]:
            assert float(recv[seg[e] + cnt[e] : seg[e + 1]].float().abs().max()) == 0.0
    # combining the dispatched rows themselves gives sum_j p_j * x[t]
    ctx.ybuf.tensor.copy_(ctx.recv.tensor)
    out, _ = ctx.combine(top_i, plan, top_p, T, gather_scalars=False)
    torch.testing.assert_close(out.float(), x.float() * top_p.sum(-1, keepdim=True), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("T,E,k,K,N", [(512, 8, 2, 256, 384), (1000, 4, 1, 128, 256)])
def test_grouped_gemm_forward_dgrad_wgrad(T, E, k, K, N):
    from nanotron_b200.ops import moe_fused

    top_p, top_i, counts = _routing(T, E, k, seed=1, empty_expert=1)
    ctx = moe_fused.get_context(None, K, T, k, E)
    plan = ctx.make_plan(counts, top_i)
    seg, cnt, cap = plan.seg_off.tolist(), counts.tolist(), ctx.cap_rows
    torch.manual_seed(0)
    a = torch.zeros(cap, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.zeros(cap, N, device="cuda", dtype=torch.bfloat16)
    for e in range(E):
        a[seg[e] : seg[e] + cnt[e]] = torch.randn(cnt[e], K, device="cuda").to(torch.bfloat16)
        dy[seg[e] : seg[e] + cnt[e]] = torch.randn(cnt[e], N, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, K, N, device="cuda") * 0.1).to(torch.bfloat16)  # [E, in, out]
    out = ctx.grouped(a, w, True, plan)  # a @ w[e]
    dgrad = ctx.grouped(dy, w, False, plan)  # dy @ w[e]^T: w read as [E, rows = K, reduction = N]
    dw = ctx.grouped_wgrad(a, dy, w, plan)  # bf16, zero for experts without rows
    w.main_grad = torch.full((E, K, N), 0.5, device="cuda", dtype=torch.float32)
    assert ctx.grouped_wgrad(a, dy, w, plan) is None
    torch.cuda.synchronize()
    ctx.check()
    for e in range(E):
        r = slice(seg[e], seg[e] + cnt[e])
        ae, dye, we = a[r].float(), dy[r].float(), w[e].float()
        if cnt[e]:
            torch.testing.assert_close(out[r].float(), ae @ we, atol=3e-2, rtol=2e-2)
            torch.testing.assert_close(dgrad[r].float(), dye @ we.t(), atol=3e-2, rtol=2e-2)
        exp_dw = ae.t() @ dye
        torch.testing.assert_close(dw[e].float(), exp_dw, atol=0.15, rtol=2e-2)
        torch.testing.assert_close(w.main_grad[e], exp_dw + 0.5, atol=1e-2, rtol=1e-3)


def _layer_pair(h=256, inter=128, E=16, k=2, shared=True):
    import nanotron_b200.config as c
    from nanotron_b200.nn.moe import Qwen2MoELayer
    from nanotron_b200.parallel import ParallelContext

    single_process_env()
    ctx = ParallelContext(1, 1, 1)
    cfg = tiny_qwen_config(hidden_size=h, intermediate_size=2 * h, moe_config=c.MoEConfig(num_experts=E, top_k=k, moe_intermediate_size=inter, shared_expert_intermediate_size=2 * inter, enable_shared_expert=shared, router_aux_loss_coef=0.01))
    torch.manual_seed(0)
    layer = Qwen2MoELayer(cfg, None, tp_pg=ctx.tp_pg, ep_pg=None).cuda()
    for name, p in layer.named_parameters():
        torch.nn.init.normal_(p, std=0.05)
    layer = layer.to(torch.bfloat16)
    layer.router.weight.data = layer.router.weight.data.float()
    return ctx, layer


def test_fused_moe_layer_matches_pytorch_path():
    from nanotron_b200.nn import moe

    ctx, layer = _layer_pair()
    T, h = 384, 256
    x = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(T, h, device="cuda", dtype=torch.bfloat16)
    results = {}
    for fused in (False, True):
        moe.FUSED_EXPERTS = fused
        for p in layer.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        out = layer(xi)
        (out["hidden_states"].float() * g.float()).sum().add(out["aux_loss"].float()).backward()
        torch.cuda.synchronize()
        results[fused] = (out["hidden_states"].detach().float(), xi.grad.float(), layer.router.weight.grad.float().clone(),
                          layer.experts.merged_gate_up_proj.grad.float().clone(), layer.experts.merged_down_proj.grad.float().clone())
    moe.FUSED_EXPERTS = True
    names = ["out", "dx", "d router", "d gate_up", "d down"]
    for n, a, b in zip(names, results[True], results[False]):
        err = (a - b).abs().max() / b.abs().max().clamp(min=1e-6)
        assert err < 3e-2, (n, float(err))
    ctx.destroy()
