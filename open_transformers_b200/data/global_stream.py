"""The canonical token stream and its per-rank view.

``GlobalStream`` is a pure function of (seed, manifests, weights, seq_len, eos): documents are drawn
source by source with ONE mixing RNG keyed on ``[seed]`` only, each followed by the separator token,
and the concatenation is cut into consecutive windows of ``seq_len + 1`` tokens. No rank or world
size enters, so every topology - and the single-device replay - sees the same windows.

``ShardedWindowView`` is what a training process iterates: it walks the same stream by document
LENGTHS only, and reads token payloads just for the windows of the micro-batches its (virtual)
ranks own (micro-batch m of a step belongs to rank m % V). Its checkpoint state is the global
stream position, identical on every rank (reference src/pretrain/data/global_stream.py:38-476).
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Iterator

import numpy as np

from ..train.batch_schedule import iter_step_plans, owner_rank
from .manifest import SourceManifest
from .mix_sampler import SourceWalker


@dataclasses.dataclass
class GlobalStreamState:
    consumed_documents_per_source: dict[str, int]
    epoch_per_source: dict[str, int]
    mix_rng_state: dict | None = None
    carry_over: list[int] = dataclasses.field(default_factory=list)
    windows_emitted: int = 0

    def to_json(self) -> dict:
        d = dataclasses.asdict(self)
        return d

    @classmethod
    def from_json(cls, d: dict) -> "GlobalStreamState":
        return cls(**d)


class _Core:
    """Shared machinery: walkers, mixing RNG, and a queue of not-yet-consumed pieces.
    piece = ("doc", source, shard, local, start, length) | ("lit", tokens ndarray)"""

    def __init__(self, manifests, manifest_dirs, weights, seq_len, seed, eos_id, state: GlobalStreamState | None, index_only: bool):
        if not (len(manifests) == len(manifest_dirs) == len(weights)):
            raise ValueError("manifests, directories and weights must have the same length")
        w = np.asarray(weights, dtype=np.float64)
        if w.sum() <= 0:
            raise ValueError("source weights must sum to a positive number")
        self.weights = w / w.sum()
        self.seq_len, self.eos = seq_len, int(eos_id)
        self.rng = np.random.default_rng(np.array([seed], dtype=np.uint64))
        consumed = state.consumed_documents_per_source if state else {}
        epochs = state.epoch_per_source if state else {}
        self.walkers = [SourceWalker(m, d, seed, 0, 1, consumed.get(m.name, 0), epochs.get(m.name, 0), index_only=index_only)
                        for m, d in zip(manifests, manifest_dirs)]
        self.pieces: deque = deque()
        self.buffered = 0
        if state and state.carry_over:
            self._push(("lit", np.asarray(state.carry_over, dtype=np.int64)), len(state.carry_over))
        if state and state.mix_rng_state is not None:
            self.rng.bit_generator.state = state.mix_rng_state
        self.windows_emitted = state.windows_emitted if state else 0
        self._eos_lit = np.asarray([self.eos], dtype=np.int64)

    def _push(self, piece, n):
        self.pieces.append(piece)
        self.buffered += n

    def refill(self) -> None:
        src = int(self.rng.choice(len(self.walkers), p=self.weights))
        shard, local = self.walkers[src].next_document_ref()
        n = self.walkers[src].reader(shard).document_length(local)
        if n:
            self._push(("doc", src, shard, local, 0, n), n)
        self._push(("lit", self._eos_lit), 1)

    def cut(self, n: int) -> list:
        """Remove the next ``n`` tokens from the queue and return them as pieces."""
        while self.buffered < n:
            self.refill()
        out, need = [], n
        while need:
            p = self.pieces.popleft()
            size = p[5] if p[0] == "doc" else len(p[1])
            if size <= need:
                out.append(p)
                need -= size
            else:
                if p[0] == "doc":
                    out.append(("doc", p[1], p[2], p[3], p[4], need))
                    self.pieces.appendleft(("doc", p[1], p[2], p[3], p[4] + need, size - need))
                else:
                    out.append(("lit", p[1][:need]))
                    self.pieces.appendleft(("lit", p[1][need:]))
                need = 0
        self.buffered -= n
        self.windows_emitted += 1
        return out

    def materialise(self, pieces) -> np.ndarray:
        parts = []
        for p in pieces:
            if p[0] == "doc":
                doc = self.walkers[p[1]].reader(p[2]).document(p[3])
                parts.append(np.asarray(doc[p[4]: p[4] + p[5]], dtype=np.int64))
            else:
                parts.append(p[1])
        return np.concatenate(parts) if parts else np.empty(0, dtype=np.int64)

    def state(self) -> GlobalStreamState:
        carry = self.materialise(list(self.pieces)).tolist() if self.pieces else []
        return GlobalStreamState({w.name: w.consumed for w in self.walkers}, {w.name: w.epoch for w in self.walkers},
                                 dict(self.rng.bit_generator.state), [int(t) for t in carry], self.windows_emitted)


class GlobalStream:
    """Iterable of the canonical ``seq_len + 1`` windows (1-D int64 arrays)."""

    def __init__(self, manifests: list[SourceManifest], manifest_dirs: list[str], weights: list[float], seq_len: int, seed: int,
                 eos_id: int = 0, state: GlobalStreamState | None = None):
        self._core = _Core(manifests, manifest_dirs, weights, seq_len, seed, eos_id, state, index_only=False)

    @property
    def windows_emitted(self) -> int:
        return self._core.windows_emitted

    def state(self) -> GlobalStreamState:
        return self._core.state()

    def __iter__(self) -> Iterator[np.ndarray]:
        n = self._core.seq_len + 1
        while True:
            yield self._core.materialise(self._core.cut(n))


class ShardedWindowView:
    """Per-process view: yields, step by step, the micro-batches owned by ``ranks`` (virtual ranks of a
    world of ``world_size``). Iterating yields ``(plan, [(rank, accum_index, windows[mb, seq_len+1]), ...])``."""

    def __init__(self, manifests, manifest_dirs, weights, seq_len, seed, train, ranks, world_size, eos_id=0,
                 state: GlobalStreamState | None = None, consumed_tokens: int = 0, start_step: int = 0, index_only: bool = False):
        self._core = _Core(manifests, manifest_dirs, weights, seq_len, seed, eos_id, state, index_only=index_only)
        self.has_carry_over = bool(state and state.carry_over)  # tokens queued by an earlier step: they name no document
        self.train, self.world_size = train, world_size
        self.ranks = [ranks] if isinstance(ranks, int) else list(ranks)
        self._consumed_tokens, self._step = consumed_tokens, start_step

    def state(self) -> GlobalStreamState:
        return self._core.state()

    @property
    def position(self) -> tuple[int, int, int]:
        return self._step, self._consumed_tokens, self._core.windows_emitted

    def __iter__(self):
        mb, n = self.train.micro_batch_size, self._core.seq_len + 1
        mine = set(self.ranks)
        for plan in iter_step_plans(self._consumed_tokens, self._core.windows_emitted, self.train, start_step=self._step):
            out = []
            for m in range(plan.microbatches):
                r = owner_rank(m, world_size=self.world_size)
                cuts = [self._core.cut(n) for _ in range(mb)]
                if r in mine:
                    out.append((r, m // self.world_size, np.stack([self._core.materialise(c) for c in cuts])))
            self._consumed_tokens += plan.tokens_this_step
            self._step += 1
            yield plan, out

    def stream_position(self) -> dict:
        """Where the stream stands, in the terms a checkpoint's ``global_stream.json`` records (payload-free: also for
        index-only walks, whose carry-over tokens cannot be materialised)."""
        c = self._core
        return {"consumed_documents_per_source": {w.name: w.consumed for w in c.walkers},
                "epoch_per_source": {w.name: w.epoch for w in c.walkers}, "windows_emitted": c.windows_emitted}

    def walk_step_spans(self, until_step: int):
        """Per optimizer step below ``until_step``: ``(plan, spans)`` with one span ``(global_window, source, shard, document,
        first token, end token)`` per document piece of the step's windows, in stream order, without reading token payloads
        (reference src/pretrain/data/global_stream.py, ``walk_step_spans``; used by the step -> document map)."""
        mb, n = self.train.micro_batch_size, self._core.seq_len + 1
        for plan in iter_step_plans(self._consumed_tokens, self._core.windows_emitted, self.train, start_step=self._step):
            if plan.step >= until_step:
                return
            spans = []
            for _ in range(plan.microbatches * mb):
                gw = self._core.windows_emitted
                for p in self._core.cut(n):
                    if p[0] == "doc":
                        spans.append((gw, self._core.walkers[p[1]].name, p[2], p[3], p[4], p[4] + p[5]))
            self._consumed_tokens += plan.tokens_this_step
            self._step += 1
            yield plan, spans

    def walk_doc_refs(self, n_steps: int):
        """(step, microbatch, slot, source, shard, local, start, length) for every document piece of the next
        ``n_steps`` steps, without reading token payloads (used by the doc map and the shard fetcher)."""
        mb, n = self.train.micro_batch_size, self._core.seq_len + 1
        for plan in iter_step_plans(self._consumed_tokens, self._core.windows_emitted, self.train, start_step=self._step):
            if plan.step >= self._step + n_steps:
                return
            for m in range(plan.microbatches):
                for slot in range(mb):
                    for p in self._core.cut(n):
                        if p[0] == "doc":
                            yield (plan.step, m, slot, self._core.walkers[p[1]].name, p[2], p[3], p[4], p[5])
