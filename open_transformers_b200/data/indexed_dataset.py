"""Megatron-compatible indexed token dataset: ``<prefix>.bin`` (raw token ids) + ``<prefix>.idx``.

.idx: 8-byte magic ``MMIDIDX\\0`` | uint64 version (1) | uint8 dtype code | int64 num_documents |
int64 token_count | int64 doc_offsets[N+1] (token offsets, with end sentinel) | int64 byte_offsets[N+1].
Same bytes as the reference's shards (src/pretrain/data/indexed_dataset.py:9-52), so either
framework reads the other's data.
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

MAGIC = b"MMIDIDX\0"
VERSION = 1
DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16, 9: np.uint32}
_CODE_OF = {np.dtype(v): k for k, v in DTYPE_CODES.items()}
CODE_BY_DTYPE = _CODE_OF
_HEAD = struct.Struct("<8sQBqq")


class IndexedDatasetReader:
    """mmap view of one shard. ``index_only=True`` reads the .idx alone (document lengths without
    touching the .bin) - enough to walk the canonical stream and find out which shards a step needs."""

    def __init__(self, prefix: str | Path, index_only: bool = False):
        self.prefix = Path(prefix)
        raw = Path(str(self.prefix) + ".idx").read_bytes()
        if len(raw) < _HEAD.size:
            raise ValueError("%s.idx: truncated header" % self.prefix)
        magic, version, code, ndocs, ntok = _HEAD.unpack_from(raw, 0)
        if magic != MAGIC:
            raise ValueError("%s.idx: bad magic %r" % (self.prefix, magic))
        if version != VERSION:
            raise ValueError("%s.idx: unsupported version %d" % (self.prefix, version))
        if code not in DTYPE_CODES:
            raise ValueError("%s.idx: unknown dtype code %d" % (self.prefix, code))
        self.dtype = np.dtype(DTYPE_CODES[code])
        self.num_documents, self.token_count = int(ndocs), int(ntok)
        need = _HEAD.size + 16 * (ndocs + 1)
        if len(raw) < need:
            raise ValueError("%s.idx: expected %d bytes, found %d" % (self.prefix, need, len(raw)))
        self.doc_offsets = np.frombuffer(raw, dtype="<i8", count=ndocs + 1, offset=_HEAD.size)
        self.byte_offsets = np.frombuffer(raw, dtype="<i8", count=ndocs + 1, offset=_HEAD.size + 8 * (ndocs + 1))
        self._tokens = None
        if not index_only:
            path = Path(str(self.prefix) + ".bin")
            self._tokens = np.memmap(path, dtype=self.dtype, mode="r") if path.stat().st_size else np.empty(0, self.dtype)

    def __len__(self) -> int:
        return self.num_documents

    def document_length(self, i: int) -> int:
        return int(self.doc_offsets[i + 1] - self.doc_offsets[i])

    def document(self, i: int) -> np.ndarray:
        if self._tokens is None:
            raise RuntimeError("%s opened index-only: token payload unavailable" % self.prefix)
        if not 0 <= i < self.num_documents:
            raise IndexError(i)
        return self._tokens[int(self.doc_offsets[i]): int(self.doc_offsets[i + 1])]

    def __iter__(self):
        for i in range(self.num_documents):
            yield self.document(i)


class IndexedDatasetWriter:
    def __init__(self, prefix: str | Path, dtype=np.uint32):
        self.prefix = Path(prefix)
        self.dtype = np.dtype(dtype)
        if self.dtype not in _CODE_OF:
            raise ValueError("unsupported token dtype %s" % self.dtype)
        self.prefix.parent.mkdir(parents=True, exist_ok=True)
        self._bin = open(str(self.prefix) + ".bin", "wb")
        self._offsets = [0]

    def add_document(self, tokens) -> None:
        arr = np.asarray(tokens)
        if arr.ndim != 1:
            raise ValueError("a document is a 1-D token array")
        if arr.size and (arr.min() < 0 and self.dtype.kind == "u" or arr.max() > np.iinfo(self.dtype).max):
            raise ValueError("token id out of range for %s" % self.dtype)
        self._bin.write(arr.astype(self.dtype, copy=False).tobytes())
        self._offsets.append(self._offsets[-1] + int(arr.size))

    @property
    def num_documents(self) -> int:
        return len(self._offsets) - 1

    @property
    def token_count(self) -> int:
        return self._offsets[-1]

    def finalize(self) -> None:
        if self._bin.closed:
            return
        self._bin.close()
        off = np.asarray(self._offsets, dtype="<i8")
        with open(str(self.prefix) + ".idx", "wb") as f:
            f.write(_HEAD.pack(MAGIC, VERSION, _CODE_OF[self.dtype], self.num_documents, self.token_count))
            f.write(off.tobytes())
            f.write((off * self.dtype.itemsize).astype("<i8").tobytes())

    close = finalize

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finalize()
