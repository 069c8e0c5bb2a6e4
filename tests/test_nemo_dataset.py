"""Megatron-format datasets: file round trip, GPT sample index (numpy statement == C++ helper, samples tile the token
stream of each epoch), train/valid/test split arithmetic, blending proportions."""
import numpy as np
import pytest

from nanotron_b200.data.nemo_dataset import (BlendableDataset, MemoryEfficientBlendableDataset, MMapIndexedDataset, get_datasets_weights_and_num_samples,
                                             get_train_valid_test_split_, make_builder)
from nanotron_b200.data.nemo_dataset.indexed_dataset import data_file_path, index_file_path


def _write(tmp_path, name, docs, vocab=1000):
    prefix = str(tmp_path / name)
    b = make_builder(data_file_path(prefix), vocab_size=vocab)
    for d in docs:
        b.add_item(np.asarray(d))
        b.end_document()
    b.finalize(index_file_path(prefix))
    return prefix


def _docs(n, seed, lo=3, hi=40, vocab=1000):
    rng = np.random.RandomState(seed)
    return [rng.randint(1, vocab, size=rng.randint(lo, hi)).tolist() for _ in range(n)]


def test_indexed_dataset_round_trip_and_merge(tmp_path):
    docs = _docs(25, 0)
    prefix = _write(tmp_path, "a", docs)
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 25 and ds.sizes.tolist() == [len(d) for d in docs] and ds.doc_idx.tolist() == list(range(26))
    for i in (0, 7, 24):
        assert ds[i].tolist() == docs[i]
    assert ds.get(3, offset=2, length=4).tolist() == docs[3][2:6]
    assert [x.tolist() for x in ds[2:5]] == docs[2:5]
    other = _write(tmp_path, "b", _docs(5, 1))
    merged = str(tmp_path / "m")
    b = make_builder(data_file_path(merged), vocab_size=1000)
    b.merge_file_(prefix)
    b.merge_file_(other)
    b.finalize(index_file_path(merged))
    m = MMapIndexedDataset(merged)
    assert len(m) == 30 and m[27].tolist() == MMapIndexedDataset(other)[2].tolist()
    import pickle

    assert pickle.loads(pickle.dumps(ds))[5].tolist() == docs[5]


def test_sample_idx_numpy_statement_matches_cpp_helper():
    from nanotron_b200.data.nemo_dataset import helpers
    from nanotron_b200.data.nemo_dataset.gpt_dataset import _build_sample_idx

    rng = np.random.RandomState(3)
    sizes = rng.randint(1, 50, size=200).astype(np.int32)
    for epochs, seq, extra, drop in [(1, 16, 1, True), (3, 33, 1, True), (2, 20, 0, True), (2, 17, 1, False)]:
        doc_idx = np.tile(np.arange(200, dtype=np.int32), epochs)
        rng.shuffle(doc_idx)
        tpe = int(sizes.sum())
        a = helpers.build_sample_idx(sizes, doc_idx, seq, epochs, tpe, drop, extra)
        b = _build_sample_idx(sizes, doc_idx, seq, epochs, tpe, drop, extra)
        assert np.array_equal(np.asarray(a), b), (epochs, seq, extra, drop)


def test_gpt_dataset_samples_tile_the_epoch_stream(tmp_path):
    from nanotron_b200.data.nemo_dataset import GPTDataset

    docs = _docs(60, 5)
    prefix = _write(tmp_path, "c", docs)
    ds = MMapIndexedDataset(prefix)
    seq = 32
    total = sum(len(d) for d in docs)
    num_samples = (2 * total - 1) // seq  # two full epochs
    g = GPTDataset(None, None, "train", prefix, np.arange(60, dtype=np.int32), ds, num_samples, seq, seed=7)
    assert len(g) == num_samples
    stream = np.concatenate([np.asarray(docs[d]) for d in g.doc_idx])
    inv = np.argsort(g.shuffle_idx)  # sample j of the un-shuffled order sits at position inv[j]
    for j in (0, 1, len(g) // 2, len(g) - 1):
        sample = g[int(inv[j])]["input_ids"]
        assert sample.shape == (seq + 1,) and sample.dtype == np.int64
        assert sample.tolist() == stream[j * seq : j * seq + seq + 1].tolist()
    # cached index maps are reused
    g2 = GPTDataset(None, None, "train", prefix, np.arange(60, dtype=np.int32), ds, num_samples, seq, seed=7)
    assert np.array_equal(g2.shuffle_idx, g.shuffle_idx)
    # two epochs: every document appears exactly twice in the shuffled document order
    assert sorted(g.doc_idx.tolist()) == sorted(list(range(60)) * 2)


def test_split_arithmetic_and_weight_normalisation():
    assert get_train_valid_test_split_("949,50,1", 1000) == [0, 949, 999, 1000]
    assert get_train_valid_test_split_("98/1/1", 200) == [0, 196, 198, 200]
    assert get_train_valid_test_split_("1", 10) == [0, 10, 10, 10]
    prefixes, weights, n = get_datasets_weights_and_num_samples([3, "a", 1, "b"], 1000)
    assert prefixes == ["a", "b"] and weights == [0.75, 0.25] and n == [754, 252]
    _, _, n3 = get_datasets_weights_and_num_samples([1, "a", 1, "b"], [100, 10, 0])
    assert n3 == [[51, 6, 0], [51, 6, 0]]


class _Range:
    def __init__(self, n, tag):
        self.n, self.tag = n, tag

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        assert 0 <= i < self.n
        return (self.tag, i)


def test_blendable_datasets_follow_the_weights():
    from nanotron_b200.data.nemo_dataset.blendable_dataset import _blend_numpy

    a, b, c = _Range(1000, "a"), _Range(1000, "b"), _Range(1000, "c")
    blend = BlendableDataset([a, b, c], [0.5, 0.3, 0.2], 1000)
    counts = {t: 0 for t in "abc"}
    seen = {t: [] for t in "abc"}
    for i in range(1000):
        t, j = blend[i]
        counts[t] += 1
        seen[t].append(j)
    assert abs(counts["a"] - 500) <= 1 and abs(counts["b"] - 300) <= 1 and abs(counts["c"] - 200) <= 1
    assert all(seen[t] == list(range(len(seen[t]))) for t in "abc")  # each dataset is read sequentially
    idx, sidx, cnt = _blend_numpy(np.asarray([0.5, 0.3, 0.2]), 1000)
    assert np.array_equal(idx, blend.dataset_index) and np.array_equal(sidx, blend.dataset_sample_index)
    blend.update_consumption_metrics(0, 100, 32)
    assert sum(blend.consumed_tokens.values()) == 3200
    me = MemoryEfficientBlendableDataset([a, b, c], [0.5, 0.3, 0.2], 1000, weight_bins=10)
    got = [me[i][0] for i in range(1000)]
    assert got.count("a") == 500 and got.count("b") == 300 and got.count("c") == 200


class _CharTokenizer:
    """One token per character (ids 10 ..), plus the five sentinel tokens the fill-in-the-middle transform needs."""

    def __init__(self):
        from nanotron_b200.data.nemo_dataset.gpt_dataset import EOD, FIM_MIDDLE, FIM_PAD, FIM_PREFIX, FIM_SUFFIX

        self.vocab = {FIM_PREFIX: 1, FIM_MIDDLE: 2, FIM_SUFFIX: 3, FIM_PAD: 4, EOD: 0}

    def decode(self, ids):
        return "".join(chr(int(i) - 10 + ord("a")) for i in ids)

    def encode(self, text):
        return [ord(ch) - ord("a") + 10 for ch in text]


def test_fill_in_the_middle_reorders_documents_without_losing_text(tmp_path):
    from types import SimpleNamespace

    from nanotron_b200.data.nemo_dataset import GPTDataset
    from nanotron_b200.data.nemo_dataset.gpt_dataset import permute

    tok = _CharTokenizer()
    ids = dict(prefix_tok_id=1, middle_tok_id=2, suffix_tok_id=3, pad_tok_id=4)
    doc = np.asarray(tok.encode("abcdefghijklmnopqrstuvwxyz"), dtype=np.int64)
    rng = np.random.RandomState(0)
    assert permute(doc, rng, 0.0, 0.5, tok, **ids) is doc  # rate 0: untouched
    seen = set()
    for _ in range(40):
        out = permute(doc, rng, 1.0, 0.5, tok, truncate_or_pad=False, **ids)
        assert len(out) == len(doc) + 3 and sorted(out.tolist()) == sorted(doc.tolist() + [1, 2, 3])
        p, m, s = (int(np.flatnonzero(out == t)[0]) for t in (1, 2, 3))
        if out[1] == 3:  # suffix-prefix-middle order: <prefix><suffix> s <middle> p m
            seen.add("spm")
            suffix, rest = out[2:m], out[m + 1 :]
            assert p == 0 and s == 1 and tok.decode(rest) + tok.decode(suffix) == tok.decode(doc)
        else:  # prefix-suffix-middle order: <prefix> p <suffix> s <middle> m
            seen.add("psm")
            assert p == 0 and p < s < m
            assert tok.decode(out[1:s]) + tok.decode(out[m + 1 :]) + tok.decode(out[s + 1 : m]) == tok.decode(doc)
    assert seen == {"spm", "psm"}
    # keeping the length: the suffix is cut by the three sentinel tokens
    out = permute(doc, np.random.RandomState(3), 1.0, 0.0, tok, truncate_or_pad=True, **ids)
    assert len(out) == len(doc)
    # through the dataset: samples keep their length, documents stay separated, sentinels appear
    rs = np.random.RandomState(1)
    docs = [list(rs.randint(10, 36, size=int(rs.randint(12, 30)))) + [0] for _ in range(40)]
    prefix = _write(tmp_path, "fim", docs)
    cfg = SimpleNamespace(fim_rate=1.0, fim_spm_rate=0.5)
    g = GPTDataset(cfg, tok, "train", prefix, np.arange(40, dtype=np.int32), MMapIndexedDataset(prefix), 20, 48, seed=5)
    plain = GPTDataset(None, None, "train", prefix, np.arange(40, dtype=np.int32), MMapIndexedDataset(prefix), 20, 48, seed=5)
    changed = 0
    for i in range(len(g)):
        a, b = g[i]["input_ids"], plain[i]["input_ids"]
        assert a.shape == b.shape == (49,)
        changed += int(not np.array_equal(a, b))
        assert {1, 2, 3} <= set(a.tolist())
    assert changed == len(g)
