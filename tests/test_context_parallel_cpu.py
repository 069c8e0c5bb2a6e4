import torch

from helpers import run_distributed


def _check_cp_attention(variant="allgather", cp=2):
    import nanotron_b200.distributed as dist
    from nanotron_b200.ops import reference as ref
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.context_parallel.ring_attention import ring_attention
    from nanotron_b200.parallel.context_parallel.zigzag import zigzag_positions, zigzag_slice, zigzag_unshard

    ctx = ParallelContext(tensor_parallel_size=1, pipeline_parallel_size=1, data_parallel_size=1, context_parallel_size=cp)
    rank = dist.get_rank(ctx.cp_pg)
    torch.manual_seed(0)
    b, S, Hq, Hkv, D = 2, 8 * cp, 4, 2, 8
    q = torch.randn(b, S, Hq, D, dtype=torch.float64)
    k = torch.randn(b, S, Hkv, D, dtype=torch.float64)
    v = torch.randn(b, S, Hkv, D, dtype=torch.float64)
    ql, kl, vl = (zigzag_slice(t, rank, cp, dim=1).reshape(-1, t.shape[2], D).clone().requires_grad_(True) for t in (q, k, v))
    pos = zigzag_positions(S, rank, cp).unsqueeze(0).expand(b, -1)
    out = ring_attention(ql, kl, vl, cp_pg=ctx.cp_pg, position_ids=pos, variant=variant)
    # oracle: full attention on one device
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    cu = torch.arange(0, (b + 1) * S, S, dtype=torch.int32)
    full = ref.attention_varlen(qf.reshape(-1, Hq, D), kf.reshape(-1, Hkv, D), vf.reshape(-1, Hkv, D), cu, cu, causal=True).reshape(b, S, Hq, D)
    exp = zigzag_slice(full, rank, cp, dim=1).reshape(-1, Hq, D)
    torch.testing.assert_close(out, exp.to(out.dtype), atol=1e-5, rtol=1e-5)
    g = torch.randn(b, S, Hq, D, dtype=torch.float64)
    full.backward(g)
    out.backward(zigzag_slice(g, rank, cp, dim=1).reshape(-1, Hq, D))
    for local, whole in ((ql, qf), (kl, kf), (vl, vf)):
        exp_g = zigzag_slice(whole.grad, rank, cp, dim=1).reshape(local.shape)
        torch.testing.assert_close(local.grad, exp_g, atol=1e-5, rtol=1e-5)
    # round trip of the sharding helpers
    parts = [zigzag_slice(q, r, cp, dim=1) for r in range(cp)]
    assert torch.equal(zigzag_unshard(parts, dim=1), q)
    ctx.destroy()


def test_zigzag_context_parallel_attention_matches_full():
    run_distributed(_check_cp_attention, 2)


def test_send_recv_ring_variant_matches_full_attention():
    """K / V blocks passed around the group (registry names "ring", "ring_flash_triton"): forward and all three gradients
    against full attention, on 2 ranks and on 4 (blocks from lower and from higher ranks, several hops)."""
    run_distributed(_check_cp_attention, 2, variant="ring", cp=2)
    run_distributed(_check_cp_attention, 4, variant="ring", cp=4)


def test_merge_attention_states():
    from nanotron_b200.ops import reference as ref
    from nanotron_b200.parallel.context_parallel.ring_attention import merge_attention_states

    torch.manual_seed(1)
    q = torch.randn(6, 2, 8)
    k = torch.randn(10, 2, 8)
    v = torch.randn(10, 2, 8)
    cq, ck = torch.tensor([0, 6], dtype=torch.int32), torch.tensor([0, 10], dtype=torch.int32)
    full, lse = ref.attention_varlen(q, k, v, cq, ck, causal=False, return_lse=True)
    ca = torch.tensor([0, 4], dtype=torch.int32)
    cb = torch.tensor([0, 6], dtype=torch.int32)
    oa, la = ref.attention_varlen(q, k[:4], v[:4], cq, ca, causal=False, return_lse=True)
    ob, lb = ref.attention_varlen(q, k[4:], v[4:], cq, cb, causal=False, return_lse=True)
    o, l = merge_attention_states(oa, la, ob, lb)
    torch.testing.assert_close(o, full, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(l, lse, atol=1e-5, rtol=1e-5)


def _check_cp_documents(cp):
    """Packed documents under zig-zag context parallelism: attention stays inside a document although the document starts lie on
    other ranks; forward and gradients against variable-length attention over the whole batch on one device."""
    import nanotron_b200.distributed as dist
    from nanotron_b200.nn.attention import get_attention_mask
    from nanotron_b200.ops import reference as ref
    from nanotron_b200.parallel import ParallelContext
    from nanotron_b200.parallel.context_parallel.ring_attention import ring_attention
    from nanotron_b200.parallel.context_parallel.zigzag import zigzag_slice

    ctx = ParallelContext(tensor_parallel_size=1, pipeline_parallel_size=1, data_parallel_size=1, context_parallel_size=cp)
    rank = dist.get_rank(ctx.cp_pg)
    torch.manual_seed(0)
    b, S, Hq, Hkv, D = 3, 8 * cp, 4, 2, 8
    # row 0: one document; row 1: starts in the middle of a document, then two more; row 2: many short documents
    lengths = [[S], [5, S // 2, S - 5 - S // 2], [3] * (S // 3) + ([S % 3] if S % 3 else [])]
    pos = torch.stack([torch.cat([torch.arange(n) for n in row]) for row in lengths])
    pos[1, :5] += 11  # the first document of row 1 began before the row
    q = torch.randn(b, S, Hq, D, dtype=torch.float64)
    k = torch.randn(b, S, Hkv, D, dtype=torch.float64)
    v = torch.randn(b, S, Hkv, D, dtype=torch.float64)
    ql, kl, vl = (zigzag_slice(t, rank, cp, dim=1).reshape(-1, t.shape[2], D).clone().requires_grad_(True) for t in (q, k, v))
    local_pos = zigzag_slice(pos, rank, cp, dim=1).contiguous()
    out = ring_attention(ql, kl, vl, cp_pg=ctx.cp_pg, position_ids=local_pos, variant="allgather", doc_masking=True)
    again = ring_attention(ql, kl, vl, cp_pg=ctx.cp_pg, position_ids=local_pos, variant="ring", doc_masking=True)  # falls back to the variant that can mask
    assert torch.equal(out, again)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    _, cu = get_attention_mask(pos, S)
    assert cu.tolist()[:4] == [0, S, S + 5, S + 5 + S // 2]  # cut at the row starts as well
    full = ref.attention_varlen(qf.reshape(-1, Hq, D), kf.reshape(-1, Hkv, D), vf.reshape(-1, Hkv, D), cu, cu, causal=True).reshape(b, S, Hq, D)
    torch.testing.assert_close(out, zigzag_slice(full, rank, cp, dim=1).reshape(-1, Hq, D), atol=1e-6, rtol=1e-6)
    g = torch.randn(b, S, Hq, D, dtype=torch.float64)
    full.backward(g)
    out.backward(zigzag_slice(g, rank, cp, dim=1).reshape(-1, Hq, D))
    for local, whole in ((ql, qf), (kl, kf), (vl, vf)):
        torch.testing.assert_close(local.grad, zigzag_slice(whole.grad, rank, cp, dim=1).reshape(local.shape), atol=1e-6, rtol=1e-6)
    # without the flag the same call attends across documents (plain causal attention)
    plain = ring_attention(ql.detach(), kl.detach(), vl.detach(), cp_pg=ctx.cp_pg, position_ids=local_pos, variant="allgather")
    assert not torch.allclose(plain, out.detach())
    ctx.destroy()


def test_packed_documents_are_masked_under_context_parallelism():
    run_distributed(_check_cp_documents, 2, cp=2)
    run_distributed(_check_cp_documents, 4, cp=4)
