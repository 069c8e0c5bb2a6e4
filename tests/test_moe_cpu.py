"""MoE layer: routing + dispatch/combine against a dense per-token loop; expert parallelism against the single-rank layer;
auxiliary loss definition."""
import torch

from helpers import make_config, run_distributed, tiny_qwen_config


def _moe_config(**kw):
    import nanotron_b200.config as c

    return tiny_qwen_config(moe_config=c.MoEConfig(num_experts=4, top_k=2, moe_intermediate_size=16, shared_expert_intermediate_size=32, enable_shared_expert=True, router_aux_loss_coef=0.01), **kw)


def _dense_moe(layer, x):
    """Per-token loop over the chosen experts: the definition the grouped implementation must match."""
    import torch.nn.functional as F

    top_p, top_i, probs = layer.router(x)
    out = torch.zeros_like(x)
    w1, w2 = layer.experts.merged_gate_up_proj, layer.experts.merged_down_proj
    for t in range(x.shape[0]):
        for s in range(layer.top_k):
            e = int(top_i[t, s])
            h = x[t] @ w1[e]
            g, u = h.chunk(2)
            out[t] += top_p[t, s] * ((F.silu(g) * u) @ w2[e])
    counts = torch.bincount(top_i.reshape(-1).long(), minlength=layer.num_experts).float()
    aux = layer.num_experts * torch.sum(counts / top_i.numel() * probs.mean(0))
    shared = layer.shared_expert(hidden_states=x)["hidden_states"] * torch.sigmoid(layer.shared_expert_gate(x))
    return out + shared, aux


def _single_rank():
    from nanotron_b200.nn.moe import Qwen2MoELayer
    from nanotron_b200.parallel import ParallelContext

    ctx = ParallelContext(1, 1, 1)
    torch.manual_seed(0)
    layer = Qwen2MoELayer(_moe_config(), None, tp_pg=ctx.tp_pg, ep_pg=None).double()
    for p in layer.parameters():
        torch.nn.init.normal_(p, std=0.3)
    x = torch.randn(10, 32, dtype=torch.float64, requires_grad=True)
    out = layer(x)
    exp, aux = _dense_moe(layer, x)
    torch.testing.assert_close(out["hidden_states"], exp, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(out["aux_loss"], aux.to(out["aux_loss"].dtype), atol=1e-6, rtol=1e-6)
    (out["hidden_states"].sum() + out["aux_loss"]).backward()
    assert layer.router.weight.grad is not None and layer.experts.merged_down_proj.grad is not None
    ctx.destroy()


def test_moe_layer_matches_dense_loop():
    run_distributed(_single_rank, 1)


def _ep_rank():
    import nanotron_b200.distributed as dist
    from nanotron_b200.nn.moe import Qwen2MoELayer
    from nanotron_b200.parallel import ParallelContext

    ctx = ParallelContext(tensor_parallel_size=1, pipeline_parallel_size=1, data_parallel_size=2, expert_parallel_size=2)
    rank = dist.get_rank(ctx.ep_pg)
    cfg = _moe_config()
    torch.manual_seed(0)
    ref_layer = Qwen2MoELayer(cfg, None, tp_pg=ctx.tp_pg, ep_pg=None).double()
    for p in ref_layer.parameters():
        torch.nn.init.normal_(p, std=0.3)
    ep_layer = Qwen2MoELayer(cfg, None, tp_pg=ctx.tp_pg, ep_pg=ctx.ep_pg).double()
    with torch.no_grad():
        ep_layer.router.weight.copy_(ref_layer.router.weight)
        ep_layer.experts.merged_gate_up_proj.copy_(ref_layer.experts.merged_gate_up_proj[rank * 2 : rank * 2 + 2])
        ep_layer.experts.merged_down_proj.copy_(ref_layer.experts.merged_down_proj[rank * 2 : rank * 2 + 2])
        for a, b in zip(ep_layer.shared_expert.parameters(), ref_layer.shared_expert.parameters()):
            a.copy_(b)
        ep_layer.shared_expert_gate.weight.copy_(ref_layer.shared_expert_gate.weight)
    torch.manual_seed(100 + rank)  # different tokens per ep rank
    x = torch.randn(7 + rank, 32, dtype=torch.float64)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    out = ep_layer(xa)["hidden_states"]
    exp = ref_layer(xb)["hidden_states"]
    torch.testing.assert_close(out, exp, atol=1e-5, rtol=1e-4)
    g = torch.randn_like(out)
    out.backward(g)
    exp.backward(g)
    torch.testing.assert_close(xa.grad, xb.grad, atol=1e-5, rtol=1e-4)
    # expert weight gradients: sum over the ep ranks' tokens of the reference gradient for the local experts
    ref_g = ref_layer.experts.merged_down_proj.grad.clone()
    dist.all_reduce(ref_g, group=ctx.ep_pg)
    torch.testing.assert_close(ep_layer.experts.merged_down_proj.grad, ref_g[rank * 2 : rank * 2 + 2], atol=1e-5, rtol=1e-4)
    ctx.destroy()


def test_expert_parallel_matches_single_rank():
    run_distributed(_ep_rank, 2)
