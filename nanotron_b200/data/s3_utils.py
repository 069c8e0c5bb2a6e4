"""Byte-range streaming of token files from the local filesystem or S3 (capability parity: reference
src/nanotron/data/s3_utils.py:20-84).  S3 access needs ``boto3``; everything else works without it."""
from __future__ import annotations

import os
import re
from typing import Iterator, List, Optional, Tuple, Union

try:
    import boto3

    BOTO3_AVAILABLE = True
except ImportError:  # pragma: no cover - optional dependency
    boto3 = None
    BOTO3_AVAILABLE = False


def _get_s3_path_components(s3_path: str) -> Tuple[str, str]:
    bucket, _, key = str(s3_path)[len("s3://"):].replace("//", "/").partition("/")
    return bucket, key


def _get_s3_object(s3_path: str):
    if not BOTO3_AVAILABLE:
        raise ImportError("boto3 is required for s3:// paths")
    bucket, key = _get_s3_path_components(s3_path)
    return boto3.resource("s3").Object(bucket_name=bucket, key=key)


def file_size(path: str) -> int:
    path = str(path)
    return _get_s3_object(path).content_length if path.startswith("s3://") else os.path.getsize(path)


def _stream_file(file_path: str, chunk_size: int, offset: int) -> Iterator[bytes]:
    """Chunks of ``chunk_size`` bytes starting at chunk number ``offset``."""
    file_path = str(file_path)
    if file_path.startswith("s3://"):
        yield from _get_s3_object(file_path).get(Range=f"bytes={chunk_size * offset}-")["Body"].iter_chunks(chunk_size)
        return
    with open(file_path, "rb") as f:
        f.seek(chunk_size * offset)
        while True:
            chunk = f.read(chunk_size)
            if not chunk:
                return
            yield chunk


def _get_s3_file_list(s3_path: str, pattern: Optional[Union[str, "re.Pattern"]] = None, recursive: bool = True, max_recursion: int = -1) -> List[str]:
    """Full ``s3://`` paths of the objects under a prefix, filtered by an optional regular expression."""
    if not BOTO3_AVAILABLE:
        raise ImportError("boto3 is required for s3:// paths")
    if isinstance(pattern, str):
        pattern = re.compile(pattern)
    bucket, prefix = _get_s3_path_components(s3_path)
    if prefix and not prefix.endswith("/"):
        prefix += "/"
    client = boto3.client("s3")
    out, todo = [], [(prefix, 0)]
    while todo:
        cur, depth = todo.pop()
        for page in client.get_paginator("list_objects_v2").paginate(Bucket=bucket, Prefix=cur, Delimiter="/"):
            for obj in page.get("Contents", []):
                full = f"s3://{bucket}/{obj['Key']}"
                if pattern is None or pattern.match(full):
                    out.append(full)
            if recursive and (max_recursion < 0 or depth < max_recursion):
                todo += [(p["Prefix"], depth + 1) for p in page.get("CommonPrefixes", [])]
    return sorted(out)
