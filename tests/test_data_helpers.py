"""Native C++ index builders against straightforward Python restatements of the same algorithms."""
import numpy as np

from nanotron_b200.data.nemo_dataset import helpers as h


def _py_blending(weights, size):
    n = len(weights)
    counts = np.zeros(n, np.int64)
    idx, sidx = np.zeros(size, np.int16), np.zeros(size, np.int64)
    for i in range(size):
        x = max(float(i), 1.0)
        err = weights * x - counts
        d = int(np.argmax(err))  # first maximum, like the strict ">" scan
        idx[i], sidx[i] = d, counts[d]
        counts[d] += 1
    return idx, sidx, counts


def _py_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, add_extra_token=1):
    num_samples = (num_epochs * tokens_per_epoch - add_extra_token) // seq_length
    out = np.zeros((num_samples + 1, 2), np.int32)
    pos, offset = 0, 0
    for s in range(1, num_samples + 1):
        need = seq_length + add_extra_token
        while need != 0:
            avail = sizes[doc_idx[pos]] - offset
            need -= avail
            if need <= 0:
                offset += need + avail - add_extra_token
                need = 0
            else:
                pos += 1
                offset = 0
        out[s] = (pos, offset)
    return out


def test_blending_indices():
    rs = np.random.RandomState(0)
    for _ in range(5):
        w = rs.rand(4)
        w /= w.sum()
        n = 777
        di, ds, cnt = np.zeros(n, np.int16), np.zeros(n, np.int64), np.zeros(4, np.int64)
        h.build_blending_indices(di, ds, cnt, w, 4, n, False)
        e = _py_blending(w, n)
        assert np.array_equal(di, e[0]) and np.array_equal(ds, e[1]) and np.array_equal(cnt, e[2])
        assert np.abs(cnt / n - w).max() < 0.01


def test_sample_idx():
    rs = np.random.RandomState(1)
    for _ in range(5):
        ndoc = 40
        sizes = rs.randint(3, 120, size=ndoc).astype(np.int32)
        epochs = 2
        doc_idx = np.concatenate([rs.permutation(ndoc) for _ in range(epochs)]).astype(np.int32)
        got = h.build_sample_idx(sizes, doc_idx, 32, epochs, int(sizes.sum()))
        assert np.array_equal(got, _py_sample_idx(sizes, doc_idx, 32, epochs, int(sizes.sum())))


def test_span_mappings_cover_documents():
    docs = np.array([0, 3, 3, 4, 9, 12], np.int64)
    sizes = np.array([10, 20, 30, 5, 40, 40, 40, 40, 40, 7, 8, 9], np.int32)
    m = h.build_mapping(docs, sizes, 1, 1000, 64, 0.0, 1234, False, 2)
    assert m.dtype == np.uint32 and m.shape[1] == 3
    # documents 0, 3 and 4 have >= 2 sentences; every span stays inside one document
    for a, b, target in m.tolist():
        assert target == 64 and any(docs[d] <= a < b <= docs[d + 1] for d in (0, 3, 4))
    covered = sorted((a, b) for a, b, _ in m.tolist())
    assert covered[0] == (0, 3) and covered[-1] == (9, 12)
    b = h.build_blocks_mapping(docs, sizes, np.full(5, 4, np.int32), 1, 1000, 64, 99, False, True)
    assert b.shape[1] == 4 and set(b[:, 2].tolist()) == {0, 2, 3, 4}
    assert sorted(b[:, 3].tolist()) == list(range(len(b)))
    # same seed, same order
    assert np.array_equal(b, h.build_blocks_mapping(docs, sizes, np.full(5, 4, np.int32), 1, 1000, 64, 99, False, True))
