"""Megatron-style GPT pre-training dataset over memory-mapped token files (capability parity: reference
src/nanotron/data/nemo_dataset/__init__.py:42-940).

A dataset is three index arrays over an ``MMapIndexedDataset``:

* ``doc_idx``     the documents of the split, repeated for as many epochs as ``num_samples`` needs and shuffled as a whole
                  (the last epoch is shuffled on its own when it contributes fewer than 80 % of an epoch's samples, so that a
                  partial epoch is not mixed into the full ones);
* ``sample_idx``  [n + 1, 2] (position in doc_idx, token offset): sample i spans from entry i to entry i + 1, built by the C++
                  helper ``build_sample_idx``;
* ``shuffle_idx`` a permutation of the samples.

The arrays are cached as ``.npy`` next to the data (or in ``index_mapping_dir``), built by the first rank and memory-mapped by the
others.  Optional fill-in-the-middle (FIM) augmentation re-orders each document of a sample into prefix / suffix / middle with
sentinel tokens.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.data.nemo_dataset.blendable_dataset import BlendableDataset
from nanotron_b200.data.nemo_dataset.dataset_utils import get_datasets_weights_and_num_samples, get_train_valid_test_split_
from nanotron_b200.data.nemo_dataset.indexed_dataset import MMapIndexedDataset, make_indexed_dataset
from nanotron_b200.logging import log_rank
from nanotron_b200.utils import main_rank_first

logger = logging.get_logger(__name__)

FIM_PREFIX, FIM_MIDDLE, FIM_SUFFIX, FIM_PAD, EOD = "<fim_prefix>", "<fim_middle>", "<fim_suffix>", "<fim_pad>", "<|endoftext|>"


@dataclass
class SubsetSplitLog:
    name: str
    data_prefix: str
    doc_idx_filename: str
    sample_idx_filename: str
    shuffle_idx_filename: str
    tokens_per_epoch: int
    num_epochs: int
    num_samples: int
    seq_length: int


def get_indexed_dataset(data_prefix: str, skip_warmup: bool) -> MMapIndexedDataset:
    t0 = time.time()
    ds = make_indexed_dataset(data_prefix, skip_warmup)
    log_rank(f" > indexed dataset {data_prefix}: {ds.sizes.shape[0]} documents, opened in {time.time() - t0:.3f} s", logger=logger, level=logging.INFO, rank=0)
    return ds


def _num_tokens(documents: np.ndarray, sizes: np.ndarray) -> int:
    return int(np.sum(sizes[documents]))


def _num_epochs(tokens_per_epoch: int, seq_length: int, num_samples: int, add_extra_token: int = 1) -> int:
    """Smallest number of passes over the split that yields ``num_samples`` samples of ``seq_length`` (+1) tokens."""
    epochs, tokens = 0, 0
    while True:
        epochs += 1
        tokens += tokens_per_epoch
        if (tokens - add_extra_token) // seq_length >= num_samples:
            return epochs


def _build_doc_idx(documents: np.ndarray, num_epochs: int, np_rng, separate_last_epoch: bool) -> np.ndarray:
    if not separate_last_epoch or num_epochs == 1:
        doc_idx = np.tile(documents.astype(np.int32), num_epochs)
        np_rng.shuffle(doc_idx)
        return doc_idx
    head = _build_doc_idx(documents, num_epochs - 1, np_rng, False)
    tail = _build_doc_idx(documents, 1, np_rng, False)
    return np.concatenate((head, tail))


def _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last=True, add_extra_token=1) -> np.ndarray:
    """Pure-numpy statement of the C++ ``build_sample_idx`` (used by tests and when the helper library is missing)."""
    total = num_epochs * tokens_per_epoch - add_extra_token
    num_samples = total // seq_length if drop_last else -(-total // seq_length)
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    d, off = 0, 0
    for i in range(1, num_samples + 1):
        remaining = seq_length + add_extra_token
        while remaining != 0:
            length = int(sizes[doc_idx[d]]) - off
            remaining -= length
            if remaining <= 0:
                off += remaining + length - add_extra_token
                remaining = 0
            else:
                if d == len(doc_idx) - 1:
                    assert i == num_samples
                    off = int(sizes[doc_idx[d]]) - add_extra_token
                    break
                d += 1
                off = 0
        out[i] = (d, off)
    return out


def _build_shuffle_idx(num_samples: int, total_size: int, np_rng) -> np.ndarray:
    """Permutation of [0, num_samples) followed by a permutation of [num_samples, total_size)."""
    dtype = np.uint32 if total_size < np.iinfo(np.uint32).max - 1 else np.int64
    first = np.arange(num_samples, dtype=dtype)
    np_rng.shuffle(first)
    if num_samples == total_size:
        return first
    last = np.arange(num_samples, total_size, dtype=dtype)
    np_rng.shuffle(last)
    return np.concatenate((first, last))


def _build_index_mappings(name, data_prefix, documents, sizes, num_samples, seq_length, seed, parallel_context, index_mapping_dir=None, drop_last=True,
                          add_extra_token=1) -> Tuple[Tuple[np.ndarray, np.ndarray, np.ndarray], SubsetSplitLog]:
    tokens_per_epoch = _num_tokens(documents, sizes)
    num_epochs = _num_epochs(tokens_per_epoch, seq_length, num_samples, add_extra_token)
    np_rng = np.random.RandomState(seed=seed)
    base = os.path.join(index_mapping_dir, os.path.basename(data_prefix)) if index_mapping_dir is not None else data_prefix
    base += f"_{name}_indexmap_{num_samples}ns_{seq_length}sl_{seed}s"
    files = [base + s for s in ("_doc_idx.npy", "_sample_idx.npy", "_shuffle_idx.npy")]

    def build():
        if all(os.path.isfile(f) for f in files):
            return
        log_rank(" > index map files not found, building them on the first rank ...", logger=logger, level=logging.INFO, rank=0)
        if num_epochs == 1:
            separate_last_epoch = False
            from_earlier_epochs = 0
        else:
            from_earlier_epochs = ((num_epochs - 1) * tokens_per_epoch - add_extra_token) // seq_length
            last_epoch_samples = num_samples - from_earlier_epochs
            per_epoch = (tokens_per_epoch - add_extra_token) // seq_length
            assert 0 <= last_epoch_samples <= per_epoch + 1, (last_epoch_samples, per_epoch)
            separate_last_epoch = last_epoch_samples < int(0.80 * per_epoch)
        t0 = time.time()
        doc_idx = _build_doc_idx(documents, num_epochs, np_rng, separate_last_epoch)
        np.save(files[0], doc_idx, allow_pickle=True)
        try:
            from nanotron_b200.data.nemo_dataset import helpers

            sample_idx = helpers.build_sample_idx(np.ascontiguousarray(sizes, dtype=np.int32), doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last, add_extra_token)
        except (ImportError, OSError):
            sample_idx = _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, drop_last, add_extra_token)
        np.save(files[1], sample_idx, allow_pickle=True)
        n_first = from_earlier_epochs if separate_last_epoch else sample_idx.shape[0] - 1
        np.save(files[2], _build_shuffle_idx(n_first, sample_idx.shape[0] - 1, np_rng), allow_pickle=True)
        log_rank(f" > built doc / sample / shuffle index maps in {time.time() - t0:.2f} s", logger=logger, level=logging.INFO, rank=0)

    if parallel_context is not None and dist.is_available() and dist.is_initialized():
        with main_rank_first(parallel_context.world_pg):
            build()
    else:
        build()
    doc_idx, sample_idx, shuffle_idx = (np.load(f, allow_pickle=True, mmap_mode="r") for f in files)
    log = SubsetSplitLog(name=name, data_prefix=data_prefix, doc_idx_filename=files[0], sample_idx_filename=files[1], shuffle_idx_filename=files[2],
                         tokens_per_epoch=tokens_per_epoch, num_epochs=num_epochs, num_samples=sample_idx.shape[0], seq_length=seq_length)
    return (doc_idx, sample_idx, shuffle_idx), log


def permute(sample: np.ndarray, np_rng, fim_rate: float, fim_spm_rate: float, tokenizer, truncate_or_pad: bool = True, suffix_tok_id: int = None,
            prefix_tok_id: int = None, middle_tok_id: int = None, pad_tok_id: int = None, no_fim_prefix: Optional[str] = None) -> np.ndarray:
    """Fill-in-the-middle transform of one document: with probability ``fim_rate`` cut the decoded text at two random
    character positions and emit PSM (``<prefix> p <suffix> s <middle> m``) or, with probability ``fim_spm_rate``, SPM order."""
    if not np_rng.binomial(1, fim_rate):
        return sample
    text = tokenizer.decode(sample)
    if no_fim_prefix is not None and text.startswith(no_fim_prefix):
        return sample
    lo, hi = sorted(int(b) for b in np_rng.randint(low=0, high=len(text) + 1, size=2))
    enc = lambda s: np.asarray(tokenizer.encode(s), dtype=np.int64).reshape(-1)  # noqa: E731
    prefix, middle, suffix = enc(text[:lo]), enc(text[lo:hi]), enc(text[hi:])
    if truncate_or_pad:
        diff = suffix.shape[0] + prefix.shape[0] + middle.shape[0] + 3 - sample.shape[0]
        if diff > 0:
            if suffix.shape[0] <= diff:
                return sample
            suffix = suffix[: suffix.shape[0] - diff]
        elif diff < 0:
            suffix = np.concatenate([suffix, np.full((-diff,), pad_tok_id)])
    if np_rng.binomial(1, fim_spm_rate):
        return np.concatenate([[prefix_tok_id, suffix_tok_id], suffix, [middle_tok_id], prefix, middle]).astype(np.int64)
    return np.concatenate([[prefix_tok_id], prefix, [suffix_tok_id], suffix, [middle_tok_id], middle]).astype(np.int64)


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, cfg: Any, tokenizer, name: str, data_prefix: str, documents: np.ndarray, indexed_dataset: MMapIndexedDataset, num_samples: int,
                 seq_length: int, seed: int, parallel_context=None, drop_last: bool = True):
        super().__init__()
        self.name, self.indexed_dataset, self.drop_last, self.seq_length = name, indexed_dataset, drop_last, seq_length
        assert np.min(documents) >= 0 and np.max(documents) < indexed_dataset.sizes.shape[0]
        g = lambda k, d=None: getattr(cfg, k, d) if cfg is not None else d  # noqa: E731
        self.eod_mask_loss = g("eod_mask_loss", False)
        self.add_extra_token = 0 if g("no_seqlen_plus_one_input_tokens", False) else 1
        self.index_mapping_dir = g("index_mapping_dir")
        self.fim_rate, self.fim_spm_rate = g("fim_rate", 0.0), g("fim_spm_rate", 0.5)
        if not (0 <= self.fim_rate <= 1 and 0 <= self.fim_spm_rate <= 1):
            raise ValueError("FIM rates are probabilities")
        self.tokenizer = tokenizer
        if self.fim_rate > 0:
            vocab = tokenizer.vocab
            self.suffix_tok_id, self.prefix_tok_id, self.middle_tok_id, self.pad_tok_id, self.eod_tok_id = (vocab[t] for t in (FIM_SUFFIX, FIM_PREFIX, FIM_MIDDLE, FIM_PAD, EOD))
            split = g("fim_split_sample")
            self.fim_split_sample = vocab[split] if split is not None else None
            self.fragment_fim_rate = g("fragment_fim_rate", 0.5)
            self.no_fim_prefix = g("no_fim_prefix")
        self.np_rng = np.random.RandomState(seed=seed)
        if self.index_mapping_dir is not None:
            os.makedirs(self.index_mapping_dir, exist_ok=True)
        (self.doc_idx, self.sample_idx, self.shuffle_idx), self.subset_log = _build_index_mappings(
            name, data_prefix, documents, indexed_dataset.sizes, num_samples, seq_length, seed, parallel_context, index_mapping_dir=self.index_mapping_dir,
            drop_last=drop_last, add_extra_token=self.add_extra_token)

    def __len__(self) -> int:
        return self.sample_idx.shape[0] - 1  # sample i spans sample_idx[i] .. sample_idx[i + 1]

    def _get_text(self, idx: int) -> np.ndarray:
        idx = int(self.shuffle_idx[idx])
        (d0, o0), (d1, o1) = self.sample_idx[idx], self.sample_idx[idx + 1]
        d0, o0, d1, o1 = int(d0), int(o0), int(d1), int(o1)
        ds, extra = self.indexed_dataset, self.add_extra_token
        if d0 == d1:
            sample = ds.get(int(self.doc_idx[d0]), offset=o0, length=o1 - o0 + extra)
        else:
            parts = [ds.get(int(self.doc_idx[d0]), offset=o0)]
            parts += [ds.get(int(self.doc_idx[i])) for i in range(d0 + 1, d1)]
            parts.append(ds.get(int(self.doc_idx[d1]), length=o1 + extra))
            sample = np.concatenate(parts)
        want = self.seq_length + extra
        sample = np.asarray(sample, dtype=np.int64)
        if len(sample) != want:  # only the very last sample of a split that is not dropped
            sample = np.pad(sample, (0, want - len(sample)), mode="constant", constant_values=-1)
        if self.fim_rate == 0:
            return sample
        return self._fim(sample)

    # ---- fill-in-the-middle
    def _fim_doc(self, seq: np.ndarray, rate: float) -> np.ndarray:
        return permute(seq, self.np_rng, rate, self.fim_spm_rate, self.tokenizer, truncate_or_pad=False, suffix_tok_id=self.suffix_tok_id,
                       prefix_tok_id=self.prefix_tok_id, middle_tok_id=self.middle_tok_id, pad_tok_id=self.pad_tok_id, no_fim_prefix=self.no_fim_prefix)

    def _fim_fragments(self, seq: np.ndarray) -> np.ndarray:
        if self.fim_split_sample is None:
            return self._fim_doc(seq, self.fim_rate)
        cuts = np.flatnonzero(seq == self.fim_split_sample)
        if cuts.size == 0:
            return self._fim_doc(seq, self.fim_rate)
        if not self.np_rng.binomial(1, self.fim_rate):
            return seq
        out, start = [], 0
        for loc in cuts:
            if loc - start > 0:
                out += [self._fim_doc(seq[start:loc], self.fragment_fim_rate), [self.fim_split_sample]]
            start = loc + 1
        out.append(self._fim_doc(seq[start:], self.fragment_fim_rate))
        return np.concatenate(out)

    def _fim(self, sample: np.ndarray) -> np.ndarray:
        n = sample.shape[0]
        breaks = np.flatnonzero(sample == self.eod_tok_id)
        if breaks.size:
            out, start = [], 0
            for loc in breaks:
                if loc - start > 0:
                    out += [self._fim_fragments(sample[start:loc]), [self.eod_tok_id]]
                start = loc + 1
            out.append(self._fim_fragments(sample[start:]))
            sample = np.concatenate(out)
        else:
            sample = self._fim_fragments(sample)
        if sample.shape[0] > n:
            sample = sample[:n]
        elif sample.shape[0] < n:
            sample = np.concatenate([sample, np.full((n - sample.shape[0],), self.pad_tok_id)])
        return sample.astype(np.int64)

    def __getitem__(self, idx: int) -> Dict[str, np.ndarray]:
        return {"input_ids": self._get_text(idx)}


def build_dataset(cfg, tokenizer, data_prefix: List[str], num_samples: int, seq_length: int, seed, skip_warmup: bool, name: str, parallel_context=None) -> Union[GPTDataset, BlendableDataset]:
    """One prefix -> a GPTDataset over all its documents; [w0, p0, w1, p1, ...] -> a weighted blend."""

    def one(prefix: str, n: int) -> GPTDataset:
        indexed = get_indexed_dataset(prefix, skip_warmup)
        documents = np.arange(0, indexed.sizes.shape[0], dtype=np.int32)
        return GPTDataset(cfg, tokenizer, name, prefix, documents, indexed, n, seq_length, seed, parallel_context, drop_last=getattr(cfg, "drop_last", True) if cfg is not None else True)

    if len(data_prefix) == 1:
        return one(data_prefix[0], num_samples)
    prefixes, weights, per_dataset = get_datasets_weights_and_num_samples(data_prefix, num_samples)
    datasets = [one(p, n) for p, n in zip(prefixes, per_dataset)]
    return BlendableDataset(datasets, weights, num_samples, parallel_context=parallel_context, seed=seed, consumed_samples=0, dataset_name=name)


def _build_train_valid_test_datasets(cfg, tokenizer, data_prefix: str, splits_string: str, train_valid_test_num_samples, seq_length: int, seed, parallel_context,
                                     skip_warmup: bool):
    indexed = get_indexed_dataset(data_prefix, skip_warmup)
    splits = get_train_valid_test_split_(splits_string, indexed.sizes.shape[0])

    def split(i: int, name: str) -> Optional[GPTDataset]:
        if splits[i + 1] <= splits[i]:
            return None
        documents = np.arange(splits[i], splits[i + 1], dtype=np.int32)
        return GPTDataset(cfg, tokenizer, name, data_prefix, documents, indexed, train_valid_test_num_samples[i], seq_length, seed, parallel_context)

    return split(0, "train"), split(1, "valid"), split(2, "test")


def build_train_valid_test_datasets(cfg, tokenizer, data_prefix: Union[Dict, List], splits_string: str, train_valid_test_num_samples: Tuple[int, int, int],
                                    seq_length: int, seed, parallel_context=None, skip_warmup: bool = True):
    """``data_prefix`` as a dict gives separate files per split; as a list it is one prefix or a weighted list that is split by
    ``splits_string`` and blended per split."""
    if isinstance(data_prefix, dict):
        assert all(data_prefix.get(k) is not None for k in ("train", "validation", "test")), f"data prefix dictionary needs train / validation / test keys, has {list(data_prefix)}"
        names = (("train", "train"), ("validation", "valid"), ("test", "test"))
        return tuple(build_dataset(cfg, tokenizer, data_prefix[key], int(n), seq_length, seed, skip_warmup, name, parallel_context)
                     for (key, name), n in zip(names, train_valid_test_num_samples))
    if len(data_prefix) == 1:
        return _build_train_valid_test_datasets(cfg, tokenizer, data_prefix[0], splits_string, train_valid_test_num_samples, seq_length, seed, parallel_context, skip_warmup)
    prefixes, weights, per_dataset = get_datasets_weights_and_num_samples(data_prefix, list(train_valid_test_num_samples))
    parts = [_build_train_valid_test_datasets(cfg, tokenizer, p, splits_string, n, seq_length, seed, parallel_context, skip_warmup) for p, n in zip(prefixes, per_dataset)]
    out = []
    for i, name in enumerate(("train", "valid", "test")):
        dsets = [p[i] for p in parts if p[i] is not None]
        out.append(BlendableDataset(dsets, weights[: len(dsets)], train_valid_test_num_samples[i], parallel_context=parallel_context, seed=seed, consumed_samples=0,
                                    dataset_name=name) if dsets else None)
    return tuple(out)
