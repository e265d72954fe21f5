"""Step -> document map of a run (the training data explorer's table).

Walks the canonical stream by document lengths only (``manifest.yaml`` + ``.idx``, no ``.bin``, no model) and writes, for
every optimizer step, one Parquet row per document piece of each of the step's windows:

    step, global_window, microbatch, slot, frag_idx, dp_rank, source, shard_id, local_doc, tok_start, tok_end

``(source, shard_id, local_doc)`` names a document across the corpus (the key of the ``documents`` table that
``pretrain-dump-documents`` writes); ``dp_rank`` is ``owner_rank(microbatch)``, the rule the training loop uses. Files are
``step_docs-<first>-<last>.parquet`` chunks of ``chunk_steps`` steps plus ``step_docs_manifest.json``; the walk's final
stream position can be checked against a checkpoint's ``global_stream.json``.
(column set, file names and the position check follow reference src/pretrain/data/doc_map.py:28-198)
"""
from __future__ import annotations

import json
from pathlib import Path

from ..train.batch_schedule import owner_rank, window_position

COLUMNS = ("step", "global_window", "microbatch", "slot", "frag_idx", "dp_rank", "source", "shard_id", "local_doc", "tok_start", "tok_end")
_TYPES = {"step": "int32", "global_window": "int64", "microbatch": "int32", "slot": "int16", "frag_idx": "int16", "dp_rank": "int16",
          "source": "string", "shard_id": "int32", "local_doc": "int32", "tok_start": "int32", "tok_end": "int32"}
MANIFEST_NAME = "step_docs_manifest.json"


def schema():
    import pyarrow as pa

    return pa.schema([(name, getattr(pa, _TYPES[name])()) for name in COLUMNS])


def step_rows(plan, spans, *, micro_batch_size: int, dp_world_size: int) -> dict[str, list]:
    """One step's spans ``(global_window, source, shard, document, first token, end token)`` as columns; ``frag_idx`` counts
    the pieces of a window from 0."""
    cols: dict[str, list] = {c: [] for c in COLUMNS}
    window, piece = None, 0
    for gw, source, shard, local, start, end in spans:
        piece = piece + 1 if gw == window else 0
        window = gw
        microbatch, slot = window_position(gw, plan, micro_batch_size=micro_batch_size)
        for name, value in zip(COLUMNS, (plan.step, gw, microbatch, slot, piece, owner_rank(microbatch, world_size=dp_world_size), source, shard,
                                         local, start, end)):
            cols[name].append(value)
    return cols


def iter_doc_map(view, *, until_step: int, micro_batch_size: int, dp_world_size: int):
    """``(plan, columns)`` per step of an index-only view, up to (not including) ``until_step``."""
    for plan, spans in view.walk_step_spans(until_step):
        yield plan, step_rows(plan, spans, micro_batch_size=micro_batch_size, dp_world_size=dp_world_size)


class ChunkedParquet:
    """Rows gathered step by step and written as ``step_docs-<first>-<last>.parquet`` every ``chunk_steps`` steps. A chunk gets
    its name only when it is whole (written beside it as ``.part`` first), so a reader of the directory never sees half a file."""

    def __init__(self, out_dir: Path, chunk_steps: int):
        self.dir, self.every = out_dir, max(1, chunk_steps)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.files: list[str] = []
        self._cols: dict[str, list] = {c: [] for c in COLUMNS}
        self._span: list[int] = []            # [first step, last step] of what is pending

    def add(self, step: int, cols: dict[str, list]) -> bool:
        """Take one step's rows; True when that completed a chunk."""
        self._span = [self._span[0] if self._span else step, step]
        for c in COLUMNS:
            self._cols[c] += cols[c]
        if (step + 1) % self.every:
            return False
        self.flush()
        return True

    def flush(self) -> None:
        if not self._span or not self._cols["step"]:
            self._span = []
            return
        import pyarrow as pa
        import pyarrow.parquet as pq

        sch = schema()
        final = self.dir / ("step_docs-%06d-%06d.parquet" % tuple(self._span))
        part = final.with_suffix(".parquet.part")
        pq.write_table(pa.table({c: pa.array(self._cols[c], type=sch.field(c).type) for c in COLUMNS}), part, compression="zstd")
        part.replace(final)
        self.files.append(str(final))
        self._cols, self._span = {c: [] for c in COLUMNS}, []


def write_doc_map(view, out_dir: str | Path, *, until_step: int, micro_batch_size: int, dp_world_size: int, chunk_steps: int = 1000,
                  progress=None) -> dict:
    """Map every step of the view below ``until_step`` into ``out_dir``. The returned summary is the body of the manifest:
    how many steps / windows / rows (rows also per source), the files, and where the stream stood when the walk ended -
    the value a checkpoint of that step records in ``global_stream.json``. ``progress(next_step, rows_so_far)`` is called
    after each completed chunk."""
    sink = ChunkedParquet(Path(out_dir), chunk_steps)
    count = {"steps": 0, "windows": 0, "rows": 0}
    by_source: dict[str, int] = {}
    for plan, cols in iter_doc_map(view, until_step=until_step, micro_batch_size=micro_batch_size, dp_world_size=dp_world_size):
        count["steps"] += 1
        count["windows"] += plan.microbatches * micro_batch_size
        count["rows"] += len(cols["step"])
        for name in cols["source"]:
            by_source[name] = by_source.get(name, 0) + 1
        if sink.add(plan.step, cols) and progress is not None:
            progress(plan.step + 1, count["rows"])
    sink.flush()
    return {"until_step": until_step, "steps_walked": count["steps"], "windows": count["windows"], "rows": count["rows"],
            "rows_per_source": by_source, "files": sink.files, "position": view.stream_position()}


def compare_position(position: dict, global_stream_json: dict) -> list[str]:
    """Differences between the position a walk ended at and a checkpoint's ``global_stream.json``, in words; empty = they
    agree. A source named on one side only is a difference (an old file with fewer sources must not pass by accident)."""
    problems = []
    for key in ("consumed_documents_per_source", "epoch_per_source"):
        want, got = global_stream_json.get(key, {}) or {}, position.get(key, {}) or {}
        for name in sorted(set(want) | set(got)):
            if want.get(name) != got.get(name):
                problems.append("%s[%s]: walk=%s ckpt=%s" % (key, name, got.get(name), want.get(name)))
    if global_stream_json.get("windows_emitted") != position.get("windows_emitted"):
        problems.append("windows_emitted: walk=%s ckpt=%s" % (position.get("windows_emitted"), global_stream_json.get("windows_emitted")))
    return problems


def write_manifest(out_dir: str | Path, summary: dict, extra: dict | None = None) -> Path:
    path = Path(out_dir) / MANIFEST_NAME
    path.write_text(json.dumps({**summary, **(extra or {})}, indent=2))
    return path
