"""Datasets over flat files of token ids ("tokenized bytes": little-endian uint16 / uint32, one document after the other), local or
on S3 (capability parity: reference src/nanotron/data/tokenized_bytes.py:36-716).

* ``TokenizedBytesFileDataset``      one file, read as a forward stream of ``seq_len + 1`` token chunks (seeks / reopens the stream
                                      when a non-consecutive index is asked for); wraps around at the end of the file.
* ``OldTokenizedBytesFolderDataset`` a folder of such streamed files with token budgets (``max_tokens`` / ``skip_tokens``).
* ``TokenizedBytesFolderDataset``    a folder of memory-mapped files (random access, optional per-token position ids that restart
                                      at every document), the default.
* ``get_tb_datasets`` / ``get_tb_dataloader`` blend several folders with weights and wrap them in the Megatron batch sampler and
                                      the causal-LM collators.
"""
from __future__ import annotations

import fnmatch
import os
import re
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, Union

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

from nanotron_b200 import distributed as dist
from nanotron_b200 import logging
from nanotron_b200.data.nanoset import TokenFile
from nanotron_b200.data.s3_utils import _get_s3_file_list, _stream_file, file_size
from nanotron_b200.logging import human_format, log_rank

logger = logging.get_logger(__name__)


@dataclass
class TBFileDatasetLog:
    dataset_type: str
    file_path: str
    seq_len: int
    dtype: str
    skip_in_stream: bool
    num_samples: int
    num_tokens: int
    human_format_num_tokens: str
    num_epochs: int


@dataclass
class TBFolderDatasetLog:
    dataset_type: str
    folder_path: str
    filename_pattern: str
    recursive: bool
    seq_len: int
    dtype: str
    skip_in_stream: bool
    num_samples: int
    num_tokens: int
    human_format_num_tokens: str
    shuffle: bool
    seed: int
    num_epochs: int
    files_order: List[str]


@dataclass
class TrainDataLog:
    train_num_samples: int
    eval_num_samples: Optional[int]
    test_num_samples: Optional[int]
    global_batch_size: int
    sequence_length: int
    total_training_tokens: int
    human_total_train_tokens: str
    train_subset: object
    eval_subset: object
    test_subset: object


class TokenizedBytesFileDataset(Dataset):
    def __init__(self, file_path: str, seq_len: int, dtype=np.uint16, skip_in_stream: bool = True, num_samples: Optional[int] = None,
                 max_tokens: Optional[int] = None, skip_tokens: Optional[int] = None):
        self.file_path, self.seq_len, self.dtype = file_path, seq_len, dtype
        self.dtype_size = np.dtype(dtype).itemsize
        self.skip_in_stream = skip_in_stream
        self.skip_tokens = skip_tokens or 0
        num_tokens = file_size(file_path) // self.dtype_size - self.skip_tokens
        self._len = max(0, (min(max_tokens, num_tokens) if max_tokens else num_tokens) // (seq_len + 1))
        self._stream = None
        self._last = None  # index served by the last __getitem__
        n_tok = self._len * (seq_len + 1)
        self.subset_log = TBFileDatasetLog(dataset_type=type(self).__name__, file_path=file_path, seq_len=seq_len, dtype=np.dtype(dtype).name, skip_in_stream=skip_in_stream,
                                           num_samples=self._len, num_tokens=n_tok, human_format_num_tokens=human_format(n_tok),
                                           num_epochs=num_samples // self._len if num_samples and self._len else 0)

    def _open_stream(self, index: int):
        """Generator of int64 tensors of ``seq_len + 1`` tokens starting at sample ``index``.  The skipped prefix is expressed in
        bytes, so it does not have to be a whole number of samples."""
        chunk = self.dtype_size * (self.seq_len + 1)
        skip_bytes = self.skip_tokens * self.dtype_size

        def gen():
            for raw in _stream_from_byte(self.file_path, skip_bytes + index * chunk, chunk):
                if len(raw) != chunk:
                    return
                yield torch.as_tensor(np.frombuffer(raw, self.dtype).astype(np.int64))

        return gen()

    def _next(self):
        delay = 0.01
        while True:
            try:
                return next(self._stream)
            except StopIteration:
                raise IndexError(f"{self.file_path}: stream ended at sample {self._last}")
            except Exception:
                if delay >= 2.0:
                    logger.error("Giving up on re-establishing stream.")
                    raise
                time.sleep(delay)
                self._stream = self._open_stream(self._last)
                delay *= 2

    def __getitem__(self, item: int) -> Dict[str, torch.Tensor]:
        i = item % len(self)  # wrap around: asking past the end starts the next epoch of this file
        if self._stream is not None and self.skip_in_stream and self._last is not None and i > self._last:
            while self._last < i - 1:  # consume the samples in between instead of reopening
                self._last += 1
                self._next()
        elif self._stream is None or i != (self._last if self._last is not None else -2) + 1:
            self._stream = self._open_stream(i)
        self._last = i
        return {"input_ids": self._next()}

    def __len__(self) -> int:
        return self._len


def _stream_from_byte(path: str, start_byte: int, chunk: int):
    """Chunks of ``chunk`` bytes from byte ``start_byte`` on (local seek or an S3 range request)."""
    if str(path).startswith("s3://"):
        from nanotron_b200.data.s3_utils import _get_s3_object

        yield from _get_s3_object(path).get(Range=f"bytes={start_byte}-")["Body"].iter_chunks(chunk)
        return
    if start_byte % chunk == 0:
        yield from _stream_file(path, chunk, start_byte // chunk)
        return
    with open(path, "rb") as f:
        f.seek(start_byte)
        while True:
            raw = f.read(chunk)
            if not raw:
                return
            yield raw


def _list_files(folder_path: str, pattern, recursive: bool) -> List[str]:
    if folder_path.startswith("s3://"):
        return _cached_s3_listing(folder_path, pattern, recursive)
    out = []
    for root, _, files in os.walk(folder_path):
        for f in files:
            full = os.path.join(root, f)
            ok = pattern is None or (pattern.match(full) if isinstance(pattern, re.Pattern) else fnmatch.fnmatch(f, pattern))
            if ok:
                out.append(full)
        if not recursive:
            break
    return sorted(out)


def _cached_s3_listing(folder_path: str, pattern, recursive: bool) -> List[str]:
    """Listing a large prefix takes minutes and every rank needs it: the result is kept in
    ``$NANOTRON_CACHE (default ~/.cache/nanotron_b200)/s3_listings/<hash>.json`` and reused until ``FORCE_UPDATE_CACHE_S3=1`` asks for
    a fresh one (capability parity: reference src/nanotron/data/tokenized_bytes.py:313-360)."""
    import hashlib
    import json

    cache_dir = os.path.join(os.path.expanduser(os.environ.get("NANOTRON_CACHE", "~/.cache/nanotron_b200")), "s3_listings")
    key = hashlib.md5(f"{folder_path}:{getattr(pattern, 'pattern', pattern)}:{recursive}".encode()).hexdigest()
    cache_file = os.path.join(cache_dir, f"{key}.json")
    if os.environ.get("FORCE_UPDATE_CACHE_S3", "0") != "1" and os.path.exists(cache_file):
        try:
            with open(cache_file) as f:
                return json.load(f)["files"]
        except (OSError, ValueError, KeyError):
            pass  # unreadable cache: list again
    files = _get_s3_file_list(folder_path, pattern, recursive)
    try:
        os.makedirs(cache_dir, exist_ok=True)
        tmp = f"{cache_file}.{os.getpid()}.tmp"
        with open(tmp, "w") as f:
            json.dump({"folder": folder_path, "files": files}, f)
        os.replace(tmp, cache_file)  # atomic: concurrent ranks never read a half-written file
    except OSError:
        pass
    return files


class OldTokenizedBytesFolderDataset(Dataset):
    def __init__(self, folder_path: str, seq_len: int, filename_pattern: Union[str, "re.Pattern", None] = None, recursive: bool = True, dtype=np.uint16,
                 skip_in_stream: bool = True, num_samples: Optional[int] = None, max_tokens: Optional[int] = None, skip_tokens: Optional[int] = None,
                 shuffle: bool = False, seed: int = 42):
        self.folder_path = folder_path
        if isinstance(filename_pattern, str):
            filename_pattern = re.compile(filename_pattern)
        self.filename_pattern = filename_pattern
        paths = _list_files(folder_path, filename_pattern, recursive)
        if not paths:
            raise FileNotFoundError(f'No files matching "{filename_pattern}" found in {folder_path}')
        self.files: List[TokenizedBytesFileDataset] = []
        budget, to_skip = max_tokens, skip_tokens or 0
        for p in paths:
            f = TokenizedBytesFileDataset(p, seq_len, dtype=dtype, skip_in_stream=skip_in_stream, max_tokens=budget, skip_tokens=to_skip)
            if to_skip:
                to_skip = max(0, to_skip - len(f) * (seq_len + 1))
                if to_skip > 0:
                    continue  # the whole file falls into the skipped prefix
            self.files.append(f)
            if budget:
                budget -= len(f) * (seq_len + 1)
                if budget <= 0:
                    break
        if shuffle:
            order = np.random.default_rng(seed).permutation(len(self.files))
            self.files = [self.files[i] for i in order]
        self.lens = np.cumsum([0] + [len(f) for f in self.files]).tolist()
        self.current_file = 0
        n = self.lens[-1]
        self.subset_log = TBFolderDatasetLog(dataset_type=type(self).__name__, folder_path=folder_path, filename_pattern=str(filename_pattern), recursive=recursive,
                                             seq_len=seq_len, dtype=np.dtype(dtype).name, skip_in_stream=skip_in_stream, num_samples=n, num_tokens=n * (seq_len + 1),
                                             human_format_num_tokens=human_format(n * (seq_len + 1)), shuffle=shuffle, seed=seed,
                                             num_epochs=num_samples // n if num_samples and n else 0, files_order=[str(f.file_path) for f in self.files])

    def __getitem__(self, item: int):
        i = item % len(self)
        while not (self.lens[self.current_file] <= i < self.lens[self.current_file + 1]):  # files are visited in order most of the time
            self.current_file = (self.current_file + 1) % len(self.files)
        return self.files[self.current_file][i - self.lens[self.current_file]]

    def __len__(self) -> int:
        return self.lens[-1]


class TokenizedBytesFolderDataset(Dataset):
    """Memory-mapped ``*.ds`` files of a folder as one sample sequence.  ``folder_read_path`` reads the same relative files from
    another root (e.g. a local mirror of an S3 prefix); ``max_tokens`` truncates the folder."""

    def __init__(self, folder_path: str, seq_len: int, filename_pattern: Optional[str] = None, recursive: bool = True, token_size: int = 2,
                 max_tokens: Optional[int] = None, shuffle: bool = False, seed: int = 42, return_positions: bool = False, eos_token_id: Optional[int] = None,
                 skip_in_stream: bool = True, num_samples: Optional[int] = None, folder_read_path: Optional[str] = None, force_update_cache: bool = False):
        if return_positions and not eos_token_id:
            log_rank("return_positions=True without an eos_token_id: positions come from the .index files (or fail if there are none)", logger=logger, level=logging.WARNING, rank=0)
        self.folder_path = folder_path
        read_root = folder_read_path or folder_path
        if read_root.startswith("s3://"):
            raise ValueError("memory-mapped token folders must be local: give folder_read_path pointing at a local mirror, or use use_old_brrr_dataloader for streaming")
        paths = _list_files(read_root, filename_pattern or "*.ds", recursive)
        if not paths:
            raise FileNotFoundError(f"no token files match {filename_pattern or '*.ds'} in {read_root}")
        if shuffle:
            order = np.random.default_rng(seed).permutation(len(paths))
            paths = [paths[i] for i in order]
        self.files: List[TokenFile] = []
        budget = max_tokens
        for p in paths:
            f = TokenFile(p, seq_len, token_size, return_positions, eos_token_id)
            f.file_path = p
            if budget is not None:
                f.num_samples = min(f.num_samples, max(0, budget // (seq_len + 1)))
                budget -= f.num_samples * (seq_len + 1)
            if f.num_samples > 0:
                self.files.append(f)
            if budget is not None and budget <= 0:
                break
        self.lens = np.cumsum([0] + [len(f) for f in self.files]).tolist()
        n = self.lens[-1] if self.lens else 0
        dtype = np.uint16 if token_size == 2 else np.uint32 if token_size == 4 else np.uint64
        self.subset_log = TBFolderDatasetLog(dataset_type=type(self).__name__, folder_path=folder_path, filename_pattern=str(filename_pattern), recursive=recursive,
                                             seq_len=seq_len, dtype=np.dtype(dtype).name, skip_in_stream=skip_in_stream, num_samples=n, num_tokens=n * (seq_len + 1),
                                             human_format_num_tokens=human_format(n * (seq_len + 1)), shuffle=shuffle, seed=seed,
                                             num_epochs=num_samples // n if num_samples and n else 0, files_order=[str(f.file_path) for f in self.files])

    def __len__(self) -> int:
        return self.lens[-1] if self.lens else 0

    def __getitem__(self, i: int):
        i = i % len(self)
        k = int(np.searchsorted(self.lens, i, side="right")) - 1
        return self.files[k][i - self.lens[k]]


def build_dataset(dataset_folder: str, seq_length: int, token_size: int, return_positions: bool = False, eos_token_id: Optional[int] = None,
                  use_old_brrr_dataloader: bool = False, skip_in_stream: bool = True, num_samples: Optional[int] = None, max_tokens: Optional[int] = None,
                  skip_tokens: Optional[int] = None, shuffle: Optional[bool] = False, seed: Optional[int] = 6, folder_read_path: Optional[str] = None):
    """One dataset from a folder of token files (streamed with ``use_old_brrr_dataloader``, memory-mapped otherwise)."""
    if use_old_brrr_dataloader:
        if folder_read_path:
            log_rank(f"Ignoring folder_read_path={folder_read_path} because use_old_brrr_dataloader is True", logger=logger, level=logging.WARNING, rank=0)
        return OldTokenizedBytesFolderDataset(dataset_folder, seq_length, filename_pattern=".*\\.ds$", skip_in_stream=skip_in_stream, max_tokens=max_tokens,
                                              num_samples=num_samples, skip_tokens=skip_tokens, shuffle=shuffle, seed=seed, dtype=np.uint16 if token_size == 2 else np.uint32)
    return TokenizedBytesFolderDataset(folder_path=dataset_folder, filename_pattern="*.ds", seq_len=seq_length, recursive=False, token_size=token_size, max_tokens=max_tokens,
                                       shuffle=shuffle, return_positions=return_positions, eos_token_id=eos_token_id, seed=seed, skip_in_stream=skip_in_stream,
                                       num_samples=num_samples, folder_read_path=folder_read_path)


def get_tb_datasets(config, sequence_length: int, global_batch_size: int, train_steps: int, current_iteration: int, parallel_context, eos_token_id: Optional[int] = None,
                    shuffle: bool = False, seed: int = 6, consumed_samples: int = 0, consumed_tokens_per_dataset_folder: Optional[Dict[str, int]] = None,
                    last_stages_consumed_tokens_per_dataset_folder: Optional[Dict[str, int]] = None) -> Tuple[Dataset, TrainDataLog]:
    """All folders of a ``NanosetDatasetsArgs`` blended by ``dataset_weights`` into ``train_steps * global_batch_size`` samples.
    Samples already consumed by earlier stages shift each folder's starting point."""
    from nanotron_b200.data.nemo_dataset import BlendableDataset

    max_tokens = config.dataset_max_tokens or [None] * len(config.dataset_folder)
    train_num_samples = train_steps * global_batch_size
    offsets = {k: v // sequence_length for k, v in (last_stages_consumed_tokens_per_dataset_folder or {}).items()}
    read_paths = config.dataset_read_path
    if isinstance(read_paths, str):
        read_paths = [read_paths]
    datasets = [
        build_dataset(folder, sequence_length, token_size=config.token_size_in_bytes, return_positions=config.return_positions, eos_token_id=eos_token_id,
                      use_old_brrr_dataloader=config.use_old_brrr_dataloader, skip_in_stream=config.skip_in_stream, max_tokens=mt, num_samples=train_num_samples,
                      shuffle=shuffle, seed=seed, folder_read_path=read_paths[i] if read_paths else None)
        for i, (folder, mt) in enumerate(zip(config.dataset_folder, max_tokens))
    ]
    weights = config.dataset_weights or [1] * len(datasets)
    if read_paths:
        # a mirror holds only part of each folder: check that the files the remaining steps will touch are present
        w = np.asarray(weights, dtype=np.float64) / np.sum(weights)
        for i, d in enumerate(datasets):
            start = int(consumed_samples * w[i]) + offsets.get(d.folder_path, 0)
            end = start + int((train_steps - current_iteration) * global_batch_size * w[i])
            assert int(train_steps * global_batch_size * w[i]) <= len(d), f"not enough data for dataset {i} ({d.folder_path})"
            for k, f in enumerate(d.files):
                if max(start, d.lens[k]) < min(end, d.lens[k + 1]):
                    assert os.path.exists(f.file_path), f"dataset {i} ({d.folder_path}) will need {f.file_path}, which does not exist"
    blend = BlendableDataset(datasets, weights, train_num_samples, parallel_context=parallel_context, seed=seed,
                             consumed_tokens_per_dataset_folder=consumed_tokens_per_dataset_folder, offsets_in_samples=offsets)
    log = TrainDataLog(train_num_samples=train_num_samples, eval_num_samples=None, test_num_samples=None, global_batch_size=global_batch_size, sequence_length=sequence_length,
                       total_training_tokens=train_num_samples * sequence_length, human_total_train_tokens=human_format(train_num_samples * sequence_length),
                       train_subset=blend.subset_log, eval_subset=None, test_subset=None)
    return blend, log


def get_tb_dataloader(dataset, sequence_length: int, micro_batch_size: int, global_batch_size: int, cfg, num_workers: int, consumed_samples: int, num_samples: int,
                      parallel_context, input_pp_rank: int, output_pp_rank: int, dataloader_drop_last: bool = True, dataloader_pin_memory: bool = True,
                      use_position_ids: bool = False, use_doc_masking: bool = False) -> DataLoader:
    """Megatron batch sampler (resumable by ``consumed_samples``) + causal-LM collator over a token dataset; pipeline ranks that
    neither feed inputs nor compute the loss iterate an empty stand-in of the same length."""
    from nanotron_b200.data.clm_collator import DataCollatorForCLM, DataCollatorForCLMWithPositionIds
    from nanotron_b200.data.dataloader import get_dataloader_worker_init
    from nanotron_b200.data.samplers import EmptyInfiniteDataset, MegatronPretrainingSampler

    if dist.get_rank(parallel_context.pp_pg) not in (input_pp_rank, output_pp_rank):
        dataset = EmptyInfiniteDataset(length=len(dataset))
    dp_rank, dp_size = dist.get_rank(parallel_context.dp_pg), parallel_context.dp_pg.size()
    sampler = MegatronPretrainingSampler(total_samples=num_samples, consumed_samples=consumed_samples, micro_batch_size=micro_batch_size, data_parallel_rank=dp_rank,
                                         data_parallel_size=dp_size, drop_last=dataloader_drop_last, global_batch_size=global_batch_size,
                                         pad_samples_to_global_batch_size=getattr(cfg, "pad_samples_to_global_batch_size", False))
    if use_position_ids:
        collator = DataCollatorForCLMWithPositionIds(sequence_length=sequence_length, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank,
                                                     parallel_context=parallel_context, use_doc_masking=use_doc_masking)
    else:
        collator = DataCollatorForCLM(sequence_length=sequence_length, input_pp_rank=input_pp_rank, output_pp_rank=output_pp_rank, parallel_context=parallel_context)
    return DataLoader(dataset, batch_sampler=sampler, collate_fn=collator, num_workers=num_workers, pin_memory=dataloader_pin_memory and torch.cuda.is_available(),
                      worker_init_fn=get_dataloader_worker_init(dp_rank=dp_rank), persistent_workers=num_workers > 0)
