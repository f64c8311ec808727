"""Indexed datasets whose files live in an S3 bucket.

The index (``.idx``) is small and is downloaded once into a local cache directory; the data (``.bin``) file is read
by byte range through an in-memory window of ``bin_chunk_nbytes`` bytes, because every request has a fixed cost that
does not depend on its size.  Behaviour follows the reference's reader (galvatron/core/runtime/datasets/megatron/
utils_s3.py:13-164, indexed_dataset.py:427-503).  The client is any object with boto3's ``download_file``,
``head_object`` and ``get_object(Bucket=, Key=, Range=)`` methods; without one ``boto3.client("s3")`` is created,
which needs the ``boto3`` package and network access.
"""
from __future__ import annotations

import os
from typing import NamedTuple, Optional, Tuple

import numpy as np

S3_PREFIX = "s3://"


class S3Config(NamedTuple):
    path_to_idx_cache: str                    # local directory for downloaded .idx files
    bin_chunk_nbytes: int = 256 * 1024 * 1024  # size of the in-memory window over the .bin object


def is_s3_path(path: str) -> bool:
    return path.startswith(S3_PREFIX)


def parse_s3_path(path: str) -> Tuple[str, str]:
    """``s3://bucket/some/key`` -> ``("bucket", "some/key")``"""
    if not is_s3_path(path):
        raise ValueError("%r is not an S3 path" % path)
    bucket, _, key = path[len(S3_PREFIX):].partition("/")
    return bucket, key


def default_client():
    try:
        import boto3
    except ModuleNotFoundError as e:  # pragma: no cover - depends on the environment
        raise RuntimeError("reading %s* paths needs the boto3 package (or pass a client object)" % S3_PREFIX) from e
    return boto3.client("s3")


def object_exists(client, path: str) -> bool:
    bucket, key = parse_s3_path(path)
    try:
        client.head_object(Bucket=bucket, Key=key)
    except Exception as e:
        code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
        if code in ("404", "NoSuchKey", "NotFound") or isinstance(e, KeyError):
            return False
        raise
    return True


def maybe_download_file(s3_path: str, local_path: str, client=None) -> None:
    """Fetch the object unless the file is already there.  With ``torch.distributed`` initialised global rank 0
    downloads first, then the first rank of every other node (ranks that do not share rank 0's file system)."""
    import torch

    distributed = torch.distributed.is_available() and torch.distributed.is_initialized()
    rank = torch.distributed.get_rank() if distributed else 0
    per_node = max(1, torch.cuda.device_count()) if distributed else 1
    local_rank = rank % per_node

    def fetch():
        cl = client if client is not None else default_client()
        os.makedirs(os.path.dirname(local_path) or ".", exist_ok=True)
        bucket, key = parse_s3_path(s3_path)
        cl.download_file(bucket, key, local_path)

    if not os.path.exists(local_path) and rank == 0:
        fetch()
    if distributed:
        torch.distributed.barrier()
    if not os.path.exists(local_path) and local_rank == 0:
        fetch()
    if distributed:
        torch.distributed.barrier()
    if not os.path.exists(local_path):
        raise FileNotFoundError(local_path)


class S3BinReader:
    """Byte-range reader with one cached window.  A miss loads the aligned block that contains ``offset`` (extended
    if the request runs past its end)."""

    def __init__(self, bin_path: str, bin_chunk_nbytes: int, client=None):
        if bin_chunk_nbytes <= 0:
            raise ValueError("bin_chunk_nbytes must be positive")
        self._client = client if client is not None else default_client()
        self._bucket, self._key = parse_s3_path(bin_path)
        self._chunk = int(bin_chunk_nbytes)
        self._cache: Optional[bytes] = None
        self._start = self._end = 0
        self.requests = 0   # number of range requests sent (for tests and logging)

    def read(self, dtype, count: int, offset: int) -> np.ndarray:
        dtype = np.dtype(dtype)
        size = count * dtype.itemsize
        if self._cache is None or offset < self._start or offset + size > self._end:
            start = (offset // self._chunk) * self._chunk
            end = max(start + self._chunk, offset + size)
            body = self._client.get_object(Bucket=self._bucket, Key=self._key,
                                           Range="bytes=%d-%d" % (start, end - 1))["Body"]
            self._cache = body.read()
            self._start, self._end = start, start + len(self._cache)   # a short read at the object's end is fine
            self.requests += 1
            if offset + size > self._end:
                raise EOFError("%s/%s: bytes %d..%d are past the end of the object" %
                               (self._bucket, self._key, offset, offset + size))
        lo = offset - self._start
        return np.frombuffer(self._cache[lo:lo + size], dtype=dtype)

    def close(self):
        close = getattr(self._client, "close", None)
        if close is not None:
            close()
