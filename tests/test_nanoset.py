import numpy as np

from nanotron_b200.data.nanoset import Nanoset, TokenFolderDataset


def _write(folder, name, docs, token_size=2):
    import os

    os.makedirs(folder, exist_ok=True)
    dtype = np.uint16 if token_size == 2 else np.uint32
    path = os.path.join(folder, name)
    np.concatenate([np.asarray(d, dtype=dtype) for d in docs]).tofile(path)
    np.cumsum([len(d) for d in docs]).astype(np.uint64).tofile(path + ".index")
    return path


def test_token_files_and_positions(tmp_path):
    docs = [list(range(1, 8)), list(range(100, 105)), list(range(200, 230))]
    _write(str(tmp_path / "a"), "0.ds", docs)
    ds = TokenFolderDataset(str(tmp_path / "a"), seq_len=8, token_size=2, return_positions=True)
    flat = np.concatenate([np.asarray(d) for d in docs])
    assert len(ds) == (len(flat) - 1) // 8
    s0 = ds[0]
    assert s0["input_ids"].tolist() == flat[:9].tolist()
    # 7-token document then a 5-token document: positions restart at index 7
    assert s0["positions"].tolist() == [0, 1, 2, 3, 4, 5, 6, 0, 1]
    s1 = ds[1]
    assert s1["input_ids"].tolist() == flat[8:17].tolist()
    assert s1["positions"].tolist() == [1, 2, 3, 4, 0, 1, 2, 3, 4]


def test_nanoset_blend_follows_weights(tmp_path):
    rs = np.random.RandomState(0)
    _write(str(tmp_path / "a"), "0.ds", [rs.randint(0, 1000, size=4000).tolist()])
    _write(str(tmp_path / "b"), "0.ds", [rs.randint(0, 1000, size=4000).tolist()])
    ns = Nanoset([str(tmp_path / "a"), str(tmp_path / "b")], sequence_length=16, token_size=2, train_split_num_samples=600, dataset_weights=[0.75, 0.25], return_positions=True)
    assert len(ns) == 600
    share = (ns.dataset_index == 0).mean()
    assert abs(share - 0.75) < 0.03
    item = ns[5]
    assert item["input_ids"].shape == (17,) and item["positions"].shape == (17,)
    stats = ns.get_consumption_stats()
    assert sum(v["tokens"] for v in stats.values()) == 16
