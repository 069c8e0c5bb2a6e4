"""Mask descriptions of the programmable-mask attention backend: element-wise predicate == dense mask == what the attention
oracle applies; block-sparsity summary; boundary conversions; the soft-capped score path."""
import math

import torch

from nanotron_b200.nn import flex_attention as fx
from nanotron_b200.nn.attention import ALL_ATTENTION_FUNCTIONS
from nanotron_b200.ops import reference as ref


def test_boundary_conversions_round_trip():
    off = fx.lengths_to_offsets([3, 5, 2])
    assert off.tolist() == [0, 3, 8, 10]
    ids = fx.offsets_to_doc_ids(off)
    assert ids.tolist() == [0] * 3 + [1] * 5 + [2] * 2
    assert fx.doc_ids_to_offsets(ids).tolist() == off.tolist()
    pos = torch.tensor([[0, 1, 2, 0, 1], [0, 1, 2, 3, 4]])
    assert fx.position_ids_to_offsets(pos).tolist() == [0, 3, 5, 10]
    # a row that does not start at position 0 still starts a document (rows never share one)
    pos = torch.tensor([[0, 1, 2], [3, 4, 0]])
    assert fx.position_ids_to_offsets(pos).tolist() == [0, 3, 5, 6]


def test_mask_kinds_match_oracle_masking():
    lens = [40, 25, 63]
    T = sum(lens)
    cu = fx.lengths_to_offsets(lens)
    torch.manual_seed(0)
    q, k, v = torch.randn(T, 4, 16), torch.randn(T, 2, 16), torch.randn(T, 2, 16)
    one = torch.tensor([0, T], dtype=torch.int32)
    cases = {
        "causal": ref.attention_varlen(q, k, v, one, one, causal=True),
        "full": ref.attention_varlen(q, k, v, one, one, causal=False),
        "sliding_window": ref.attention_varlen(q, k, v, one, one, causal=True, window=16),
        "document": ref.attention_varlen(q, k, v, cu, cu, causal=True),
        "sliding_window_document": ref.attention_varlen(q, k, v, cu, cu, causal=True, window=16),
    }
    for kind, exp in cases.items():
        out = ALL_ATTENTION_FUNCTIONS["flex_attention"](q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens), max_seqlen_k=max(lens), causal=True, sliding_window=16, flex_attention_mask=kind)
        torch.testing.assert_close(out, exp, atol=1e-5, rtol=1e-5)
        # the same mask, applied densely
        bm = fx.block_mask_for(kind, cu, cu, T, T, max(lens), max(lens), causal=True, sliding_window=16)
        dense = bm.dense()
        s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(2, dim=1)) / math.sqrt(16)
        p = torch.softmax(s.masked_fill(~dense, float("-inf")), -1)
        torch.testing.assert_close(torch.einsum("hqk,khd->qhd", p, v.repeat_interleave(2, dim=1)), exp, atol=1e-5, rtol=1e-5)
        f = bm.mask_mod()
        for qi, ki in [(0, 0), (39, 0), (40, 39), (41, 40), (70, 45), (127, 64), (127, 127), (100, 120), (60, 30)]:
            assert f(qi, ki) == bool(dense[qi, ki]), (kind, qi, ki)


def test_block_table_and_cache():
    cu = fx.lengths_to_offsets([256, 256])
    bm = fx.block_mask_for("document", cu, cu, 512, 512, 256, 256)
    t = bm.block_table(128)
    assert t.tolist() == [[1, 0, 0, 0], [2, 1, 0, 0], [0, 0, 1, 0], [0, 0, 2, 1]]
    assert abs(bm.sparsity(128) - 10 / 16) < 1e-6
    assert fx.block_mask_for("document", cu, cu, 512, 512, 256, 256) is bm  # cached on the boundary tensor
    a = fx.create_block_mask_cached("sliding_window", 300, 300, 50)
    assert fx.create_block_mask_cached("sliding_window", 300, 300, 50) is a
    m = fx.create_attention_mask(10, position_ids=torch.tensor([0, 1, 2, 0, 1, 2, 3, 0, 1, 2]), sliding_window=2)
    assert m.cu_seqlens_q.tolist() == [0, 3, 7, 10] and m.max_seqlen_q == 4 and m.window == 2
    assert m.dense()[5].tolist() == [False] * 4 + [True, True] + [False] * 4


def test_softcap_bounds_the_scores():
    torch.manual_seed(1)
    T = 24
    q, k, v = 10 * torch.randn(T, 2, 8), 10 * torch.randn(T, 2, 8), torch.randn(T, 2, 8)
    cu = torch.tensor([0, T], dtype=torch.int32)
    out = ALL_ATTENTION_FUNCTIONS["flex_attention"](q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=T, max_seqlen_k=T, causal=True, softcap=5.0)
    s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(8)
    s = 5.0 * torch.tanh(s / 5.0)
    keep = torch.tril(torch.ones(T, T, dtype=torch.bool))
    exp = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(~keep, float("-inf")), -1), v)
    torch.testing.assert_close(out, exp, atol=1e-5, rtol=1e-5)
    # a very large cap is no cap
    big = ALL_ATTENTION_FUNCTIONS["flex_attention"](q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=T, max_seqlen_k=T, causal=True, softcap=1e6)
    torch.testing.assert_close(big, ref.attention_varlen(q, k, v, cu, cu, causal=True), atol=1e-4, rtol=1e-4)
