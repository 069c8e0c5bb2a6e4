"""Token-file datasets: streamed single files (sequential, skipping, random access, wrap-around, token budgets), streamed and
memory-mapped folders, weighted blending of folders through ``get_tb_datasets``."""
import numpy as np
import pytest

from nanotron_b200.data.tokenized_bytes import OldTokenizedBytesFolderDataset, TokenizedBytesFileDataset, TokenizedBytesFolderDataset, build_dataset, get_tb_datasets


def _write(path, n, start=0, dtype=np.uint16):
    np.arange(start, start + n, dtype=dtype).tofile(path)


def test_file_dataset_streams_skips_and_wraps(tmp_path):
    p = str(tmp_path / "a.ds")
    _write(p, 1000)
    seq = 9
    ds = TokenizedBytesFileDataset(p, seq)
    assert len(ds) == 100
    assert ds[0]["input_ids"].tolist() == list(range(10))
    assert ds[1]["input_ids"].tolist() == list(range(10, 20))  # consecutive: same stream
    assert ds[5]["input_ids"].tolist() == list(range(50, 60))  # skip ahead inside the stream
    assert ds[2]["input_ids"].tolist() == list(range(20, 30))  # going back reopens
    assert ds[103]["input_ids"].tolist() == list(range(30, 40))  # wraps around
    assert ds[0]["input_ids"].dtype.is_floating_point is False
    budget = TokenizedBytesFileDataset(p, seq, max_tokens=55, skip_tokens=7)
    assert len(budget) == 5 and budget[0]["input_ids"].tolist() == list(range(7, 17)) and budget[4]["input_ids"].tolist() == list(range(47, 57))
    no_skip = TokenizedBytesFileDataset(p, seq, skip_in_stream=False)
    assert no_skip[3]["input_ids"].tolist() == list(range(30, 40)) and no_skip[7]["input_ids"].tolist() == list(range(70, 80))


def test_folder_datasets(tmp_path):
    for i in range(3):
        _write(str(tmp_path / f"f{i}.ds"), 205, start=1000 * i)
    (tmp_path / "notes.txt").write_text("x")
    seq = 9
    old = OldTokenizedBytesFolderDataset(str(tmp_path), seq, filename_pattern=".*\\.ds$")
    assert len(old) == 60 and old.subset_log.num_samples == 60
    assert old[0]["input_ids"].tolist() == list(range(10)) and old[20]["input_ids"].tolist() == list(range(1000, 1010)) and old[59]["input_ids"][0] == 2190
    assert old[61]["input_ids"].tolist() == list(range(10, 20))
    capped = OldTokenizedBytesFolderDataset(str(tmp_path), seq, filename_pattern=".*\\.ds$", max_tokens=250)
    assert len(capped) == 20 + 5
    mm = TokenizedBytesFolderDataset(str(tmp_path), seq, filename_pattern="*.ds", recursive=False, token_size=2)
    # memory-mapped files share the boundary token between consecutive samples: (205 - 1) // 9 = 22 samples per file
    assert len(mm) == 66 and mm[0]["input_ids"].tolist() == list(range(10)) and mm[1]["input_ids"].tolist() == list(range(9, 19))
    assert mm[22]["input_ids"].tolist() == list(range(1000, 1010))
    shuffled = TokenizedBytesFolderDataset(str(tmp_path), seq, shuffle=True, seed=3)
    assert sorted(shuffled.subset_log.files_order) == sorted(mm.subset_log.files_order)
    pos = TokenizedBytesFolderDataset(str(tmp_path), seq, return_positions=True, eos_token_id=13)
    item = pos[1]
    assert item["input_ids"].tolist() == list(range(9, 19)) and item["positions"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4]
    assert isinstance(build_dataset(str(tmp_path), seq, 2), TokenizedBytesFolderDataset)
    assert isinstance(build_dataset(str(tmp_path), seq, 2, use_old_brrr_dataloader=True), OldTokenizedBytesFolderDataset)


def test_get_tb_datasets_blends_folders(tmp_path):
    from nanotron_b200.config import NanosetDatasetsArgs

    a, b = tmp_path / "a", tmp_path / "b"
    a.mkdir()
    b.mkdir()
    _write(str(a / "x.ds"), 5000, start=0)
    _write(str(b / "y.ds"), 5000, start=30000)
    cfg = NanosetDatasetsArgs(dataset_folder=[str(a), str(b)], dataset_weights=[3, 1], token_size_in_bytes=2, return_positions=False)
    blend, log = get_tb_datasets(cfg, sequence_length=9, global_batch_size=8, train_steps=10, current_iteration=0, parallel_context=None)
    assert len(blend) == 80 and log.train_num_samples == 80 and log.total_training_tokens == 720
    firsts = [int(blend[i]["input_ids"][0]) for i in range(80)]
    assert sum(1 for f in firsts if f < 30000) == 60 and sum(1 for f in firsts if f >= 30000) == 20
    # resuming a later stage shifts the folder that was already consumed
    later, _ = get_tb_datasets(cfg, 9, 8, 10, 0, None, last_stages_consumed_tokens_per_dataset_folder={str(a): 90})
    assert int(later[0]["input_ids"][0]) == 90


class _FakeBoto3:
    """An in-memory object store with the three entry points the streaming helpers use."""

    def __init__(self, objects):
        self.objects = objects  # {(bucket, key): bytes}
        outer = self

        class _Body:
            def __init__(self, data):
                self.data = data

            def iter_chunks(self, size):
                for i in range(0, len(self.data), size):
                    yield self.data[i : i + size]

        class _Object:
            def __init__(self, bucket_name, key):
                self.data = outer.objects[(bucket_name, key)]
                self.content_length = len(self.data)

            def get(self, Range):
                start = int(Range[len("bytes=") : -1])
                return {"Body": _Body(self.data[start:])}

        class _Resource:
            Object = staticmethod(lambda bucket_name, key: _Object(bucket_name, key))

        class _Paginator:
            def paginate(self, Bucket, Prefix, Delimiter):
                keys = sorted(k for (b, k) in outer.objects if b == Bucket and k.startswith(Prefix))
                here = [k for k in keys if Delimiter not in k[len(Prefix) :]]
                below = sorted({Prefix + k[len(Prefix) :].split(Delimiter)[0] + Delimiter for k in keys if Delimiter in k[len(Prefix) :]})
                yield {"Contents": [{"Key": k} for k in here], "CommonPrefixes": [{"Prefix": p} for p in below]}

        class _Client:
            get_paginator = staticmethod(lambda name: _Paginator())

        self.resource = lambda service: _Resource()
        self.client = lambda service: _Client()


def test_byte_range_streaming_from_files_and_from_an_object_store(tmp_path, monkeypatch):
    from nanotron_b200.data import s3_utils

    payload = bytes(range(256)) * 5
    local = tmp_path / "tokens.ds"
    local.write_bytes(payload)
    assert s3_utils.file_size(str(local)) == 1280
    assert b"".join(s3_utils._stream_file(str(local), chunk_size=100, offset=0)) == payload
    assert b"".join(s3_utils._stream_file(str(local), chunk_size=100, offset=3)) == payload[300:]  # the offset counts chunks
    assert s3_utils._get_s3_path_components("s3://bucket/a//b/c.ds") == ("bucket", "a/b/c.ds")
    store = {("bucket", "data/a/000.ds"): payload, ("bucket", "data/a/001.ds"): payload[:700], ("bucket", "data/a/000.ds.index"): b"x",
             ("bucket", "data/b/deep/002.ds"): payload[:10], ("bucket", "other/003.ds"): b"zz"}
    monkeypatch.setattr(s3_utils, "boto3", _FakeBoto3(store))
    monkeypatch.setattr(s3_utils, "BOTO3_AVAILABLE", True)
    assert s3_utils.file_size("s3://bucket/data/a/001.ds") == 700
    chunks = list(s3_utils._stream_file("s3://bucket/data/a/000.ds", chunk_size=512, offset=1))
    assert b"".join(chunks) == payload[512:] and len(chunks[0]) == 512
    assert s3_utils._get_s3_file_list("s3://bucket/data", pattern=r".*\.ds$") == ["s3://bucket/data/a/000.ds", "s3://bucket/data/a/001.ds", "s3://bucket/data/b/deep/002.ds"]
    assert s3_utils._get_s3_file_list("s3://bucket/data", pattern=r".*\.ds$", max_recursion=1) == ["s3://bucket/data/a/000.ds", "s3://bucket/data/a/001.ds"]
    assert s3_utils._get_s3_file_list("s3://bucket/data/a", recursive=False) == ["s3://bucket/data/a/000.ds", "s3://bucket/data/a/000.ds.index", "s3://bucket/data/a/001.ds"]
    monkeypatch.setattr(s3_utils, "BOTO3_AVAILABLE", False)
    with pytest.raises(ImportError):
        s3_utils.file_size("s3://bucket/data/a/001.ds")


def test_token_file_streams_from_an_object_store_and_survives_a_dropped_connection(tmp_path, monkeypatch):
    from nanotron_b200.data import s3_utils

    tokens = np.arange(9 * 40, dtype=np.uint16)
    fake = _FakeBoto3({("bucket", "run/000.ds"): tokens.tobytes()})
    monkeypatch.setattr(s3_utils, "boto3", fake)
    monkeypatch.setattr(s3_utils, "BOTO3_AVAILABLE", True)
    ds = TokenizedBytesFileDataset("s3://bucket/run/000.ds", seq_len=8, skip_tokens=4)  # samples of 9 tokens after a skipped prefix
    assert len(ds) == (360 - 4) // 9
    assert ds[0]["input_ids"].tolist() == list(range(4, 13)) and ds[1]["input_ids"].tolist() == list(range(13, 22))
    assert ds[5]["input_ids"].tolist() == list(range(4 + 45, 4 + 54))  # forward jump: the samples in between are consumed from the stream
    assert ds[2]["input_ids"].tolist() == list(range(22, 31))  # backward jump: a new range request
    # the connection drops in the middle of the stream: the dataset re-opens it at the sample it was about to serve
    real_resource = fake.resource
    state = {"opened": 0}

    def flaky_resource(service):
        res = real_resource(service)

        class Wrapper:
            @staticmethod
            def Object(bucket_name, key):
                obj = res.Object(bucket_name, key)
                real_get = obj.get

                def get(Range):
                    state["opened"] += 1
                    body = real_get(Range)["Body"]
                    first = state["opened"] == 1

                    class Body:
                        def iter_chunks(self, size):
                            for n, chunk in enumerate(body.iter_chunks(size)):
                                if first and n == 2:
                                    raise ConnectionError("connection reset")
                                yield chunk

                    return {"Body": Body()}

                obj.get = get
                return obj

        return Wrapper()

    monkeypatch.setattr(fake, "resource", flaky_resource)
    fresh = TokenizedBytesFileDataset("s3://bucket/run/000.ds", seq_len=8)
    got = [fresh[i]["input_ids"].tolist() for i in range(5)]
    assert got == [list(range(9 * i, 9 * i + 9)) for i in range(5)] and state["opened"] == 2


def test_object_store_listings_are_cached_until_a_refresh_is_asked_for(tmp_path, monkeypatch):
    from nanotron_b200.data import s3_utils, tokenized_bytes

    tokens = np.arange(90, dtype=np.uint16).tobytes()
    store = {("bucket", "run/a/000.ds"): tokens, ("bucket", "run/a/001.ds"): tokens}
    monkeypatch.setattr(s3_utils, "boto3", _FakeBoto3(store))
    monkeypatch.setattr(s3_utils, "BOTO3_AVAILABLE", True)
    monkeypatch.setenv("NANOTRON_CACHE", str(tmp_path / "cache"))
    calls = {"n": 0}
    real = tokenized_bytes._get_s3_file_list

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    monkeypatch.setattr(tokenized_bytes, "_get_s3_file_list", counting)
    first = tokenized_bytes._list_files("s3://bucket/run", None, True)
    assert first == ["s3://bucket/run/a/000.ds", "s3://bucket/run/a/001.ds"] and calls["n"] == 1
    store[("bucket", "run/a/002.ds")] = tokens  # the bucket changes ...
    assert tokenized_bytes._list_files("s3://bucket/run", None, True) == first and calls["n"] == 1  # ... the cached listing is used
    monkeypatch.setenv("FORCE_UPDATE_CACHE_S3", "1")
    assert len(tokenized_bytes._list_files("s3://bucket/run", None, True)) == 3 and calls["n"] == 2
    monkeypatch.delenv("FORCE_UPDATE_CACHE_S3")
    assert len(tokenized_bytes._list_files("s3://bucket/run", None, True)) == 3 and calls["n"] == 2  # the refreshed listing was stored
    assert tokenized_bytes._list_files("s3://bucket/run", None, False) == [] and calls["n"] == 3  # another question, another entry
