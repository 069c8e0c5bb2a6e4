"""Memory-mapped token datasets in the Megatron ``.bin`` / ``.idx`` format (capability parity: reference
src/nanotron/data/nemo_dataset/indexed_dataset.py:104-344).

``<prefix>.idx`` layout: 9-byte magic ``MMIDIDX\\x00\\x00``, u64 version (1), u8 dtype code, u64 number of sequences, u64 number
of document boundaries, then int32 sizes[n], int64 byte pointers[n], int64 doc_idx[docs].  ``<prefix>.bin`` is the concatenation
of the token arrays.  Reading never copies: sequences are numpy views of one ``np.memmap``.
"""
from __future__ import annotations

import os
import struct
from typing import Optional

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


def code(dtype) -> int:
    for k, v in _DTYPES.items():
        if v == dtype:
            return k
    raise ValueError(dtype)


def best_fitting_dtype(vocab_size: Optional[int] = None):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def index_file_path(prefix_path: str) -> str:
    return prefix_path + ".idx"


def data_file_path(prefix_path: str) -> str:
    return prefix_path + ".bin"


class MMapIndexedDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, skip_warmup: bool = True):
        super().__init__()
        self._path = path
        self._open(path, skip_warmup)

    def _open(self, path: str, skip_warmup: bool):
        with open(index_file_path(path), "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError(f"{index_file_path(path)} is not an MMIDIDX index file")
            (version,) = struct.unpack("<Q", f.read(8))
            assert version == 1, version
            (dtype_code,) = struct.unpack("<B", f.read(1))
            self._dtype = _DTYPES[dtype_code]
            (self._len,) = struct.unpack("<Q", f.read(8))
            (self._doc_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        if not skip_warmup:
            for p in (index_file_path(path), data_file_path(path)):
                with open(p, "rb") as f:
                    while f.read(100 * 1024 * 1024):
                        pass
        self._index_mmap = np.memmap(index_file_path(path), mode="r", order="C")
        buf = memoryview(self._index_mmap)
        self._sizes = np.frombuffer(buf, dtype=np.int32, count=self._len, offset=offset)
        self._pointers = np.frombuffer(buf, dtype=np.int64, count=self._len, offset=offset + self._sizes.nbytes)
        self._doc_idx = np.frombuffer(buf, dtype=np.int64, count=self._doc_count, offset=offset + self._sizes.nbytes + self._pointers.nbytes)
        self._bin_mmap = np.memmap(data_file_path(path), mode="r", order="C")
        self._bin = memoryview(self._bin_mmap)

    def __getstate__(self):
        return self._path

    def __setstate__(self, state):
        self._path = state
        self._open(state, skip_warmup=True)

    def __len__(self) -> int:
        return self._len

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            return np.frombuffer(self._bin, dtype=self._dtype, count=int(self._sizes[idx]), offset=int(self._pointers[idx]))
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("slices into an indexed dataset must be contiguous")
            sizes = self._sizes[idx]
            flat = np.frombuffer(self._bin, dtype=self._dtype, count=int(sizes.sum()), offset=int(self._pointers[start]))
            return np.split(flat, np.cumsum(sizes)[:-1])
        raise TypeError(f"unexpected index type {type(idx)}")

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """Tokens [offset, offset + length) of sequence ``idx`` without touching the rest."""
        size = int(self._sizes[idx])
        if length is None:
            length = size - offset
        ptr = int(self._pointers[idx]) + offset * np.dtype(self._dtype).itemsize
        return np.frombuffer(self._bin, dtype=self._dtype, count=length, offset=ptr)

    @property
    def sizes(self) -> np.ndarray:
        return self._sizes

    @property
    def doc_idx(self) -> np.ndarray:
        return self._doc_idx

    def get_doc_idx(self):
        return self._doc_idx

    def set_doc_idx(self, doc_idx_):
        self._doc_idx = doc_idx_

    @property
    def supports_prefetch(self) -> bool:
        return False

    @staticmethod
    def exists(path: str) -> bool:
        return os.path.exists(index_file_path(path)) and os.path.exists(data_file_path(path))

    def deallocate_indexed_dataset_memory(self):
        """Drop the (optional) in-memory copies of the index; the maps stay valid."""
        self._doc_idx = self._doc_idx


def deallocate_indexed_dataset_memory(indexed_dataset):
    if isinstance(indexed_dataset, MMapIndexedDataset):
        indexed_dataset.deallocate_indexed_dataset_memory()


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file: str, dtype=np.int64):
        self._data_file = open(out_file, "wb")
        self._dtype = dtype
        self._sizes = []
        self._doc_idx = [0]

    def add_item(self, tensor):
        arr = np.asarray(tensor.numpy() if isinstance(tensor, torch.Tensor) else tensor, dtype=self._dtype)
        self._data_file.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def end_document(self):
        self._doc_idx.append(len(self._sizes))

    def merge_file_(self, another_file: str):
        other = MMapIndexedDataset(another_file)
        assert other._dtype == self._dtype
        base = len(self._sizes)
        self._sizes.extend(int(s) for s in other.sizes)
        self._doc_idx.extend(int(d) + base for d in other.doc_idx[1:])
        with open(data_file_path(another_file), "rb") as f:
            while True:
                chunk = f.read(64 * 1024 * 1024)
                if not chunk:
                    break
                self._data_file.write(chunk)

    def finalize(self, index_file: str):
        self._data_file.close()
        sizes = np.asarray(self._sizes, dtype=np.int32)
        itemsize = np.dtype(self._dtype).itemsize
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * itemsize, out=pointers[1:])
        with open(index_file, "wb") as f:
            f.write(_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", code(self._dtype)))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(self._doc_idx)))
            f.write(sizes.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self._doc_idx, dtype=np.int64).tobytes(order="C"))


def make_builder(out_file: str, vocab_size: Optional[int] = None, **_unused) -> MMapIndexedDatasetBuilder:
    return MMapIndexedDatasetBuilder(out_file, dtype=best_fitting_dtype(vocab_size))


def make_indexed_dataset(path: str, skip_warmup: bool = False) -> MMapIndexedDataset:
    if not MMapIndexedDataset.exists(path):
        raise FileNotFoundError(f"no {index_file_path(path)} / {data_file_path(path)} pair; the path prefix should not carry an extension")
    return MMapIndexedDataset(path, skip_warmup=skip_warmup)
