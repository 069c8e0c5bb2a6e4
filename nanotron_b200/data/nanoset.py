"""Pre-tokenised token-file datasets and their weighted blend (parity: reference src/nanotron/data/nanoset.py, which
reads the files through the third-party ``datatrove`` package; the reader here is in-tree).

File format (what ``datatrove``'s tokeniser writes, and ``tools/preprocess_data.py`` here): ``<name>.ds`` holds the
token ids back to back, little-endian, ``token_size`` (2 or 4) bytes each; the optional ``<name>.ds.index`` holds the
cumulative end offset (in tokens, uint64) of every document.  A sample is ``sequence_length + 1`` consecutive tokens;
consecutive samples overlap by one token.  Position ids restart at every document boundary (from the index file, or
from ``eos_token_id`` occurrences when there is no index).
"""
from __future__ import annotations

import glob
import os
import warnings
from typing import Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from nanotron_b200 import logging
from nanotron_b200.data.utils import count_dataset_indexes, normalize
from nanotron_b200.logging import log_rank

logger = logging.get_logger(__name__)


class TokenFile:
    """One ``.ds`` file, memory-mapped."""

    def __init__(self, path: str, seq_len: int, token_size: int, return_positions: bool, eos_token_id: Optional[int]):
        self.path, self.seq_len, self.token_size = path, seq_len, token_size
        self.dtype = np.uint16 if token_size == 2 else np.uint32
        n_tokens = os.path.getsize(path) // token_size
        self.num_samples = max(0, (n_tokens - 1) // seq_len)
        self.return_positions = return_positions
        self.eos_token_id = eos_token_id
        self._mm = None
        self._doc_ends = None
        idx = path + ".index"
        self._index_path = idx if os.path.exists(idx) else None

    def _tokens(self):
        if self._mm is None:
            self._mm = np.memmap(self.path, dtype=self.dtype, mode="r")
        return self._mm

    def _ends(self):
        if self._doc_ends is None and self._index_path is not None:
            self._doc_ends = np.fromfile(self._index_path, dtype=np.uint64).astype(np.int64)
        return self._doc_ends

    def __len__(self):
        return self.num_samples

    def __getitem__(self, i: int) -> Dict[str, np.ndarray]:
        if i < 0 or i >= self.num_samples:
            raise IndexError(i)
        start = i * self.seq_len
        ids = np.asarray(self._tokens()[start : start + self.seq_len + 1], dtype=np.int64)
        out = {"input_ids": ids}
        if self.return_positions:
            out["positions"] = self._positions(start, ids)
        return out

    def _positions(self, start: int, ids: np.ndarray) -> np.ndarray:
        n = len(ids)
        pos = np.arange(n, dtype=np.int64)
        ends = self._ends()
        if ends is not None:
            # document starts that fall inside (start, start+n)
            lo = np.searchsorted(ends, start, side="right")
            hi = np.searchsorted(ends, start + n, side="left")
            starts = ends[lo:hi] - start
            # offset inside the first (partial) document
            first_doc_start = ends[lo - 1] if lo > 0 else 0
            pos += start - first_doc_start
        else:
            assert self.eos_token_id is not None, "positions need an index file or an eos token id"
            starts = np.nonzero(ids[:-1] == self.eos_token_id)[0] + 1
        for s in starts:
            if 0 < s < n:
                pos[s:] -= pos[s]
        return pos


class TokenFolderDataset(torch.utils.data.Dataset):
    """All ``*.ds`` files of a folder, seen as one sequence of samples (files optionally shuffled by seed)."""

    def __init__(self, folder_path: str, seq_len: int, token_size: int = 2, shuffle: bool = False, seed: int = 42, return_positions: bool = False, eos_token_id: Optional[int] = None, filename_pattern: Optional[str] = None):
        pattern = filename_pattern or os.path.join(folder_path, "*.ds")
        paths = sorted(glob.glob(pattern))
        if not paths:
            raise FileNotFoundError(f"no token files match {pattern}")
        if shuffle:
            np.random.RandomState(seed).shuffle(paths)
        self.files = [TokenFile(p, seq_len, token_size, return_positions, eos_token_id) for p in paths]
        self.lens = np.cumsum([0] + [len(f) for f in self.files])

    def __len__(self):
        return int(self.lens[-1])

    def __getitem__(self, i: int):
        if i < 0:
            i += len(self)
        f = int(np.searchsorted(self.lens, i, side="right")) - 1
        return self.files[f][i - int(self.lens[f])]


class Nanoset(torch.utils.data.Dataset):
    """Weighted blend of token folders.  ``dataset_weights`` None: weights proportional to the folder sizes.
    The blend index is built by the native greedy builder, shuffled with ``random_seed`` and repeated for as many epochs
    as ``train_split_num_samples`` needs."""

    def __init__(self, dataset_folders: List[str], sequence_length: int, token_size: int, train_split_num_samples: int, dataset_weights: Union[List[float], None] = None, random_seed: int = 1234, eos_token_id: Optional[int] = None, return_positions: bool = True):
        if isinstance(dataset_folders, str):
            warnings.warn("dataset_folders should be of type List[str] but str was provided. Converting to List[str]")
            dataset_folders = [dataset_folders]
        self.dataset_folders = dataset_folders
        self.sequence_length = sequence_length
        self.token_size = token_size
        self.train_split_num_samples = train_split_num_samples
        self.random_seed = random_seed
        self.eos_token_id = eos_token_id
        self.return_positions = return_positions
        self.datasets = [TokenFolderDataset(f, sequence_length, token_size, shuffle=True, seed=random_seed, return_positions=return_positions, eos_token_id=eos_token_id) for f in dataset_folders]
        self.dataset_lengths = [len(d) for d in self.datasets]
        self.dataset_weights = normalize(self.dataset_lengths) if dataset_weights is None else normalize(dataset_weights)
        assert len(dataset_folders) == len(self.dataset_weights), f"Specified {len(self.dataset_weights)} weights but {len(dataset_folders)} datasets were provided."
        self.dataset_index, self.dataset_sample_index = self.build_nanoset_index()
        self.consumed = np.zeros(len(dataset_folders), dtype=np.int64)
        self.print_nanoset_info()

    def __len__(self) -> int:
        return len(self.dataset_index)

    def __getitem__(self, idx: int) -> Dict[str, np.ndarray]:
        d = int(self.dataset_index[idx])
        s = int(self.dataset_sample_index[idx]) % self.dataset_lengths[d]
        self.consumed[d] += self.sequence_length
        return self.datasets[d][s]

    def get_consumption_stats(self, consumed_samples: Optional[int] = None) -> Dict[str, Dict[str, int]]:
        """Tokens drawn from every folder.  With ``consumed_samples`` (samples of this dataset consumed by the WHOLE job so far) the
        answer comes from the sample index itself: the job walks the index in order, so the first ``consumed_samples`` entries are
        what was read, whichever rank or loader worker read them.  Without it: what this process happened to fetch (diagnostic only,
        it misses other ranks and loader workers and runs ahead by the prefetch depth)."""
        if consumed_samples is not None:
            n = min(int(consumed_samples), len(self.dataset_index))
            counts = np.bincount(np.asarray(self.dataset_index[:n], dtype=np.int64), minlength=len(self.dataset_folders))
            return {f: {"tokens": int(c) * self.sequence_length} for f, c in zip(self.dataset_folders, counts)}
        return {f: {"tokens": int(t)} for f, t in zip(self.dataset_folders, self.consumed)}

    def build_nanoset_index(self) -> Tuple[np.ndarray, np.ndarray]:
        from nanotron_b200.data.nemo_dataset.helpers import build_blending_indices

        samples_per_epoch = sum(self.dataset_lengths)
        num_epochs = int(self.train_split_num_samples / samples_per_epoch) + 1
        dataset_index = np.zeros(samples_per_epoch, dtype=np.int16)
        dataset_sample_index = np.zeros(samples_per_epoch, dtype=np.int64)
        counts = np.zeros(len(self.dataset_folders), dtype=np.int64)
        build_blending_indices(dataset_index, dataset_sample_index, counts, self.dataset_weights, len(self.dataset_folders), samples_per_epoch, False)
        np.random.RandomState(self.random_seed).shuffle(dataset_index)
        np.random.RandomState(self.random_seed).shuffle(dataset_sample_index)
        dataset_index = np.concatenate([dataset_index] * num_epochs)[: self.train_split_num_samples]
        dataset_sample_index = np.concatenate([dataset_sample_index] * num_epochs)[: self.train_split_num_samples]
        return dataset_index, dataset_sample_index

    def print_nanoset_info(self):
        log_rank(f"> Total number of samples: {len(self)}", logger=logger, level=logging.INFO, rank=0)
        log_rank(f"> Total number of tokens: {len(self) * self.sequence_length}", logger=logger, level=logging.INFO, rank=0)
        counts = count_dataset_indexes(self.dataset_index, len(self.dataset_folders))
        shares = normalize(counts).tolist()
        for i, c in enumerate(counts):
            log_rank(f">   Total number of samples from the {self.dataset_folders[i]} dataset: {c} ({round(shares[i], 2)})", logger=logger, level=logging.INFO, rank=0)
