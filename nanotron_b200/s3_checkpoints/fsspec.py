"""Thin fsspec helpers for local / remote checkpoint paths (parity: reference src/nanotron/s3_checkpoints/fsspec.py)."""
from __future__ import annotations

import contextlib
from pathlib import Path
from typing import Tuple, Union

import fsspec
from fsspec.implementations import local


def _get_filesystem_and_path(path: Union[Path, str], storage_options=None) -> Tuple[fsspec.AbstractFileSystem, str]:
    return fsspec.core.url_to_fs(str(path), **(storage_options or {}))


@contextlib.contextmanager
def fs_open(file: Union[str, Path], mode="r"):
    fs, path = _get_filesystem_and_path(file)
    with fs.open(path, mode=mode) as f:
        yield f


def fs_copy(input_file: Union[str, Path], output_file: Union[str, Path]):
    """Copy between any two fsspec locations (downloads to / uploads from the local disk as needed)."""
    import shutil

    with fs_open(input_file, mode="rb") as fi, fs_open(output_file, mode="wb") as fo:
        shutil.copyfileobj(fi, fo, length=16 << 20)  # streamed: checkpoint shards do not fit in host memory twice


def check_path_is_local(path: Union[Path, str], storage_options=None) -> bool:
    fs, _ = _get_filesystem_and_path(path, storage_options)
    return isinstance(fs, local.LocalFileSystem)
