import torch

from nanotron_b200.parallel.parameters import NanotronParameter, SlicesPair
from nanotron_b200.parallel.sharded_parameters import SplitConfig, compute_slices_pairs
from nanotron_b200.optim.flat_layout import FlatLayout


def test_slices_pair_string_round_trip():
    sp = SlicesPair(local_slices=(slice(0, 10, None), slice(None)), global_slices=(slice(20, 30, None), slice(None)))
    assert SlicesPair.from_str(str(sp)) == sp
    t = (sp, sp)
    assert SlicesPair.tuple_from_str(SlicesPair.tuple_to_str(t)) == t


def test_fused_chunk_sharding_reassembles():
    # q|k|v = 8|4|4 rows split over 2 ranks
    full = torch.arange(16 * 3).view(16, 3).float()
    chunks = (8, 4, 4)
    rebuilt = torch.zeros_like(full)
    for rank in range(2):
        local = torch.cat([full[0:8].chunk(2)[rank], full[8:12].chunk(2)[rank], full[12:16].chunk(2)[rank]])
        pairs, shape = compute_slices_pairs(tuple(local.shape), SplitConfig(split_dim=0, contiguous_chunks=chunks), rank, 2)
        assert shape == (16, 3)
        for p in pairs:
            rebuilt[p.global_slices] = local[p.local_slices]
    assert torch.equal(rebuilt, full)


def test_metadata_cannot_be_overwritten():
    p = NanotronParameter(torch.zeros(4))
    p.mark_as_sharded(global_ranks=(0, 1), local_global_slices_pairs=(), unsharded_shape=(8,))
    assert p.is_sharded and not p.is_tied
    try:
        p.mark_as_sharded(global_ranks=(0, 1), local_global_slices_pairs=(), unsharded_shape=(8,))
        raise AssertionError("expected ValueError")
    except ValueError:
        pass


def test_flat_layout_partitions_every_element_once():
    layout = FlatLayout.build([("a", 1000), ("b", 77), ("c", 5000), ("d", 3)], world=4)
    assert layout.total % (4 * 128) == 0
    table = layout.param_name_to_dp_rank_offsets()
    for name, n in [("a", 1000), ("b", 77), ("c", 5000), ("d", 3)]:
        covered = torch.zeros(n, dtype=torch.int32)
        for r, (s, e) in table[name].items():
            covered[s:e] += 1
        assert bool((covered == 1).all()), name
