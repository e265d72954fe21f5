"""Document order inside one source, and the legacy per-rank mixing sampler.

Per epoch a source's documents are visited in a permutation built from numpy ``default_rng``
streams keyed on uint64 arrays: shards are shuffled with key (seed, H(name), epoch) and the
documents of each shard with key (seed, H(name), epoch, shard_id), H = first 4 bytes of
sha256(name). Rank r of w takes entries r, r+w, r+2w... (the canonical stream uses r=0, w=1).
numpy's bit generators are the pinned source of randomness: the permutation must equal the
reference's for the same seed (src/pretrain/data/mix_sampler.py:143-215).
"""
from __future__ import annotations

import dataclasses
import hashlib
from pathlib import Path

import numpy as np

from .indexed_dataset import IndexedDatasetReader
from .manifest import SourceManifest

_PERMS: dict[tuple, np.ndarray] = {}
_READERS: dict[tuple, IndexedDatasetReader] = {}


def stable_name_hash(name: str) -> int:
    return int.from_bytes(hashlib.sha256(name.encode("utf-8")).digest()[:4], "big")


def cached_reader(prefix, index_only: bool = False) -> IndexedDatasetReader:
    key = (str(prefix), bool(index_only))
    if key not in _READERS:
        full = _READERS.get((str(prefix), False))
        _READERS[key] = full if (index_only and full is not None) else IndexedDatasetReader(prefix, index_only=index_only)
    return _READERS[key]


def clear_caches() -> None:
    _PERMS.clear()
    _READERS.clear()


class SourceWalker:
    def __init__(self, manifest: SourceManifest, manifest_dir: str, seed: int, rank: int = 0, world_size: int = 1,
                 start_consumed: int = 0, start_epoch: int = 0, index_only: bool = False):
        self.name, self.seed, self.rank, self.world_size = manifest.name, seed, rank, world_size
        base = Path(manifest_dir)
        self.readers = [cached_reader(s.prefix if Path(s.prefix).is_absolute() else base / s.prefix, index_only) for s in manifest.shards]
        counts = np.asarray([r.num_documents for r in self.readers], dtype=np.int64)
        self._counts = counts
        self._cum = np.concatenate([[0], np.cumsum(counts)])
        self.total_documents = int(self._cum[-1])
        if self.total_documents == 0:
            raise ValueError("source %s has no documents" % self.name)
        self.consumed, self.epoch = start_consumed, start_epoch
        self._perm = self._permutation(self.epoch)

    def _permutation(self, epoch: int) -> np.ndarray:
        nh = stable_name_hash(self.name)
        key = (self.seed, nh, epoch, self.total_documents, len(self.readers))
        if key not in _PERMS:
            order = np.random.default_rng(np.array([self.seed, nh, epoch], dtype=np.uint64)).permutation(len(self.readers))
            parts = []
            for sid in order:
                rng = np.random.default_rng(np.array([self.seed, nh, epoch, int(sid)], dtype=np.uint64))
                parts.append(rng.permutation(int(self._counts[sid])) + int(self._cum[sid]))
            _PERMS[key] = np.concatenate(parts)
        return _PERMS[key]

    def next_document_ref(self) -> tuple[int, int]:
        """(shard_id, index inside the shard) of the next document for this rank."""
        pos = self.consumed * self.world_size + self.rank
        if pos >= self._perm.size:
            self.epoch += 1
            self.consumed = 0
            self._perm = self._permutation(self.epoch)
            pos = self.rank
        doc = int(self._perm[pos])
        self.consumed += 1
        sid = int(np.searchsorted(self._cum, doc, side="right") - 1)
        return sid, doc - int(self._cum[sid])

    def next_document(self) -> np.ndarray:
        sid, local = self.next_document_ref()
        return self.readers[sid].document(local)

    def reader(self, shard_id: int) -> IndexedDatasetReader:
        return self.readers[shard_id]


@dataclasses.dataclass
class MixSamplerState:
    consumed_documents_per_source: dict[str, int]
    epoch_per_source: dict[str, int]
    mix_rng_state: dict | None = None
    carry_over: list[int] = dataclasses.field(default_factory=list)


class MixSampler:
    """Legacy per-rank sampler: mixing RNG keyed (seed, rank, world). Topology-dependent, kept for
    non-auditable DDP runs; the canonical stream (global_stream.py) replaces it."""

    def __init__(self, manifests, manifest_dirs, weights, seq_len, seed, rank=0, world_size=1, eos_id=0, state: MixSamplerState | None = None):
        w = np.asarray(weights, dtype=np.float64)
        self._weights = w / w.sum()
        self._seq_len, self._eos = seq_len, eos_id
        self._rng = np.random.default_rng(np.array([seed, rank, world_size], dtype=np.uint64))
        consumed = state.consumed_documents_per_source if state else {}
        epochs = state.epoch_per_source if state else {}
        self._walkers = [SourceWalker(m, d, seed, rank, world_size, consumed.get(m.name, 0), epochs.get(m.name, 0))
                         for m, d in zip(manifests, manifest_dirs)]
        self._buf: list[int] = list(state.carry_over) if state else []
        if state and state.mix_rng_state is not None:
            self._rng.bit_generator.state = state.mix_rng_state

    def state(self) -> MixSamplerState:
        return MixSamplerState({w.name: w.consumed for w in self._walkers}, {w.name: w.epoch for w in self._walkers},
                               dict(self._rng.bit_generator.state), list(self._buf))

    def __iter__(self):
        n = self._seq_len + 1
        while True:
            while len(self._buf) < n:
                src = int(self._rng.choice(len(self._walkers), p=self._weights))
                self._buf.extend(int(t) for t in self._walkers[src].next_document())
                self._buf.append(self._eos)
            out, self._buf = self._buf[:n], self._buf[n:]
            yield np.asarray(out, dtype=np.int64)
