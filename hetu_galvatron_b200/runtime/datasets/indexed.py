"""Memory-mapped indexed dataset: a flat ``.bin`` token array plus an ``.idx`` describing sequences and documents.

``.idx`` layout (little endian): magic ``b"MMIDIDX\\x00\\x00"``, ``<Q`` version (1), ``<B`` dtype code, ``<Q`` sequence
count, ``<Q`` document count, ``int32[seq]`` lengths, ``int64[seq]`` byte pointers, ``int64[doc]`` document boundaries
(indices into the sequence list, first entry 0), optionally ``int8[seq]`` modes.  Dtype codes: 1 uint8, 2 int8,
3 int16, 4 int32, 5 int64, 6 float64, 7 float32, 8 uint16.  Files written here are readable by the reference's reader
and vice versa (galvatron/core/runtime/datasets/megatron/indexed_dataset.py:38-52, :126-205, :344-503, :506-742).
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np

MAGIC = b"MMIDIDX\x00\x00"
VERSION = 1
DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
CODE_OF = {np.dtype(v): k for k, v in DTYPE_CODES.items()}


def optimal_dtype(vocab_size: Optional[int]):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def idx_path(prefix: str) -> str:
    return prefix + ".idx"


def bin_path(prefix: str) -> str:
    return prefix + ".bin"


class IndexedDatasetBuilder:
    """Append token sequences, mark document ends, then ``finalize`` to write the index."""

    def __init__(self, bin_file: str, dtype=np.int32, multimodal: bool = False):
        self.f = open(bin_file, "wb")
        self.dtype = np.dtype(dtype)
        self.lengths: List[int] = []
        self.doc_idx: List[int] = [0]
        self.modes: Optional[List[int]] = [] if multimodal else None

    def add_item(self, tokens, mode: int = 0):
        arr = np.asarray(tokens, dtype=self.dtype)
        self.f.write(arr.tobytes(order="C"))
        self.lengths.append(arr.size)
        if self.modes is not None:
            self.modes.append(mode)

    def end_document(self):
        self.doc_idx.append(len(self.lengths))

    def add_document(self, tokens, lengths: Sequence[int], modes: Optional[Sequence[int]] = None):
        arr = np.asarray(tokens, dtype=self.dtype)
        self.f.write(arr.tobytes(order="C"))
        self.lengths.extend(int(x) for x in lengths)
        self.doc_idx.append(len(self.lengths))
        if self.modes is not None and modes is not None:
            self.modes.extend(modes)

    def finalize(self, idx_file: str):
        self.f.close()
        lengths = np.asarray(self.lengths, dtype=np.int32)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(idx_file, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<Q", VERSION))
            f.write(struct.pack("<B", CODE_OF[self.dtype]))
            f.write(struct.pack("<Q", len(lengths)))
            f.write(struct.pack("<Q", len(self.doc_idx)))
            f.write(lengths.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self.doc_idx, dtype=np.int64).tobytes(order="C"))
            if self.modes is not None:
                f.write(np.asarray(self.modes, dtype=np.int8).tobytes(order="C"))


class IndexedDataset:
    """``path_prefix`` may be an ``s3://bucket/key-prefix``: the index is then downloaded into
    ``s3_config.path_to_idx_cache`` and the data file read by byte range (``runtime/datasets/s3.py``)."""

    def __init__(self, path_prefix: str, multimodal: bool = False, mmap: bool = True, s3_config=None, s3_client=None):
        self.prefix, self.multimodal = path_prefix, multimodal
        self._s3 = None
        if path_prefix.startswith("s3://"):
            from . import s3 as _s3

            if s3_config is None:
                raise ValueError("an S3 dataset needs an S3Config (where to cache the index, window size)")
            local_idx = os.path.join(s3_config.path_to_idx_cache, os.path.basename(idx_path(path_prefix)))
            _s3.maybe_download_file(idx_path(path_prefix), local_idx, s3_client)
            self._s3 = _s3.S3BinReader(bin_path(path_prefix), s3_config.bin_chunk_nbytes, s3_client)
            local_prefix, mmap = local_idx[:-len(".idx")], False
        else:
            local_prefix = path_prefix
        self._open_index(local_prefix, multimodal)
        if self._s3 is not None:
            self._bin, self._file = None, None
        elif mmap:
            self._bin = np.memmap(bin_path(path_prefix), mode="r", order="C")
            self._file = None
        else:
            self._bin, self._file = None, open(bin_path(path_prefix), "rb")

    def _open_index(self, path_prefix: str, multimodal: bool):
        with open(idx_path(path_prefix), "rb") as f:
            if f.read(9) != MAGIC:
                raise ValueError("%s is not an indexed-dataset index" % idx_path(path_prefix))
            (version,) = struct.unpack("<Q", f.read(8))
            if version != VERSION:
                raise ValueError("unsupported index version %d" % version)
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = np.dtype(DTYPE_CODES[code])
            (self.sequence_count,) = struct.unpack("<Q", f.read(8))
            (self.document_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._idx = np.memmap(idx_path(path_prefix), mode="r", order="C")
        n = self.sequence_count
        self.sequence_lengths = np.frombuffer(self._idx, dtype=np.int32, count=n, offset=offset)
        self.sequence_pointers = np.frombuffer(self._idx, dtype=np.int64, count=n, offset=offset + 4 * n)
        self.document_indices = np.frombuffer(self._idx, dtype=np.int64, count=self.document_count, offset=offset + 12 * n)
        self.sequence_modes = None
        if multimodal:
            self.sequence_modes = np.frombuffer(self._idx, dtype=np.int8, count=n, offset=offset + 12 * n + 8 * self.document_count)

    @staticmethod
    def exists(prefix: str, s3_client=None) -> bool:
        if prefix.startswith("s3://"):
            from . import s3 as _s3

            cl = s3_client if s3_client is not None else _s3.default_client()
            return _s3.object_exists(cl, idx_path(prefix)) and _s3.object_exists(cl, bin_path(prefix))
        return os.path.exists(idx_path(prefix)) and os.path.exists(bin_path(prefix))

    def __len__(self):
        return self.sequence_count

    def _read(self, pointer: int, count: int):
        if self._s3 is not None:
            return self._s3.read(self.dtype, count, pointer)
        if self._bin is not None:
            return np.frombuffer(self._bin, dtype=self.dtype, count=count, offset=pointer)
        self._file.seek(pointer)
        return np.frombuffer(self._file.read(count * self.dtype.itemsize), dtype=self.dtype)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(len(self)))]
        return self.get(int(i))

    def get(self, i: int, offset: int = 0, length: Optional[int] = None):
        n = int(self.sequence_lengths[i])
        length = n - offset if length is None else length
        seq = self._read(int(self.sequence_pointers[i]) + offset * self.dtype.itemsize, length)
        if self.sequence_modes is not None:
            return seq, self.sequence_modes[i]
        return seq
