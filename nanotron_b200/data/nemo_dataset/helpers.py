"""Python face of the native dataset index builders (``nanotron_b200/data/csrc/index_helpers.cpp``).

Function names and signatures match the reference's pybind11 module ``helpers``
(reference src/nanotron/data/nemo_dataset/helpers.cpp) so dataset code can call either.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_int32, c_int64, c_uint64, c_void_p
from pathlib import Path

import numpy as np

_LIB = None
_PATH = Path(__file__).resolve().parent.parent / "libntb_dataidx.so"


def _lib():
    global _LIB
    if _LIB is None:
        if not _PATH.exists():
            from nanotron_b200.ops.build import build_data_helpers

            build_data_helpers()
        L = ctypes.CDLL(str(_PATH))
        L.ntb_build_blending_indices.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64]
        L.ntb_build_blending_indices.restype = None
        L.ntb_sample_idx_num_samples.argtypes = [c_int32, c_int32, c_int64, c_int, c_int]
        L.ntb_sample_idx_num_samples.restype = c_int64
        L.ntb_build_sample_idx.argtypes = [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int64, c_int, c_int, c_void_p]
        L.ntb_build_sample_idx.restype = None
        L.ntb_build_mapping.argtypes = [c_void_p, c_int64, c_void_p, c_int32, c_uint64, c_int32, c_double, c_int32, c_int32, c_void_p]
        L.ntb_build_mapping.restype = c_void_p
        L.ntb_build_blocks_mapping.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_uint64, c_int32, c_int32, c_int, c_void_p]
        L.ntb_build_blocks_mapping.restype = c_void_p
        L.ntb_rows_copy_and_free.argtypes = [c_void_p, c_void_p, c_int]
        L.ntb_rows_copy_and_free.restype = None
        _LIB = L
    return _LIB


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def build_blending_indices(dataset_index, dataset_sample_index, dataset_num_samples, weights, num_datasets: int, size: int, verbose: bool = False):
    """In place: fills ``dataset_index`` (int16) and ``dataset_sample_index`` (int64); ``dataset_num_samples`` (int64) is
    the running per-dataset count (start it at zeros)."""
    assert dataset_index.dtype == np.int16 and dataset_sample_index.dtype == np.int64 and dataset_num_samples.dtype == np.int64
    assert dataset_index.flags.c_contiguous and dataset_sample_index.flags.c_contiguous and dataset_num_samples.flags.c_contiguous
    w = _c(weights, np.float64)
    _lib().ntb_build_blending_indices(dataset_index.ctypes.data, dataset_sample_index.ctypes.data, dataset_num_samples.ctypes.data, w.ctypes.data, int(num_datasets), int(size))
    if verbose:
        ratios = dataset_num_samples / max(1, size)
        print("> sample ratios:", ", ".join(f"dataset {i}: input {w[i]:.4f} achieved {ratios[i]:.4f}" for i in range(num_datasets)))


def build_sample_idx(sizes, doc_idx, seq_length: int, num_epochs: int, tokens_per_epoch: int, drop_last: bool = True, add_extra_token: int = 1) -> np.ndarray:
    sizes = _c(sizes, np.int32)
    doc_idx = _c(doc_idx, np.int32)
    L = _lib()
    n = L.ntb_sample_idx_num_samples(seq_length, num_epochs, tokens_per_epoch, int(drop_last), add_extra_token)
    out = np.empty((n + 1, 2), dtype=np.int32)
    L.ntb_build_sample_idx(sizes.ctypes.data, doc_idx.ctypes.data, len(doc_idx), seq_length, num_epochs, tokens_per_epoch, int(drop_last), add_extra_token, out.ctypes.data)
    return out


def _collect(handle, rows: int, width: int, wide: bool) -> np.ndarray:
    out = np.empty((rows, width), dtype=np.uint64 if wide else np.uint32)
    _lib().ntb_rows_copy_and_free(handle, out.ctypes.data, int(wide))
    return out


def build_mapping(docs, sizes, num_epochs: int, max_num_samples: int, max_seq_length: int, short_seq_prob: float, seed: int, verbose: bool = False, min_num_sent: int = 2) -> np.ndarray:
    docs = _c(docs, np.int64)
    sizes = _c(sizes, np.int32)
    rows = c_int64(0)
    h = _lib().ntb_build_mapping(docs.ctypes.data, len(docs), sizes.ctypes.data, num_epochs, int(max_num_samples), max_seq_length, float(short_seq_prob), seed, min_num_sent, ctypes.byref(rows))
    return _collect(h, rows.value, 3, sizes.size > np.iinfo(np.uint32).max)


def build_blocks_mapping(docs, sizes, titles_sizes, num_epochs: int, max_num_samples: int, max_seq_length: int, seed: int, verbose: bool = False, use_one_sent_blocks: bool = False) -> np.ndarray:
    docs = _c(docs, np.int64)
    sizes = _c(sizes, np.int32)
    titles = _c(titles_sizes, np.int32)
    rows = c_int64(0)
    h = _lib().ntb_build_blocks_mapping(docs.ctypes.data, len(docs), sizes.ctypes.data, titles.ctypes.data, num_epochs, int(max_num_samples), max_seq_length, seed, int(use_one_sent_blocks), ctypes.byref(rows))
    return _collect(h, rows.value, 4, sizes.size > np.iinfo(np.uint32).max)
