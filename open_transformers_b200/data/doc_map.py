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


def _write_chunk(cols: dict[str, list], out_dir: Path, first: int, last: int) -> str:
    import pyarrow as pa
    import pyarrow.parquet as pq

    sch = schema()
    table = pa.table({name: pa.array(cols[name], type=sch.field(name).type) for name in COLUMNS})
    path = out_dir / ("step_docs-%06d-%06d.parquet" % (first, last))
    part = path.with_suffix(".parquet.part")       # a reader never sees a half-written chunk
    pq.write_table(table, part, compression="zstd")
    part.replace(path)
    return str(path)


def write_doc_map(view, out_dir: str | Path, *, until_step: int, micro_batch_size: int, dp_world_size: int, chunk_steps: int = 1000,
                  progress=None) -> dict:
    """Walk the view's steps below ``until_step`` into Parquet chunks under ``out_dir``. Returns the summary that goes into
    the manifest: steps, windows, rows (total and per source), files, and the stream position at the end of the walk."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    pending: dict[str, list] = {c: [] for c in COLUMNS}
    files, per_source = [], {}
    rows = windows = steps = 0
    first = last = None
    for plan, cols in iter_doc_map(view, until_step=until_step, micro_batch_size=micro_batch_size, dp_world_size=dp_world_size):
        first = plan.step if first is None else first
        last = plan.step
        steps += 1
        rows += len(cols["step"])
        windows += plan.microbatches * micro_batch_size
        for name in cols["source"]:
            per_source[name] = per_source.get(name, 0) + 1
        for c in COLUMNS:
            pending[c].extend(cols[c])
        if (plan.step + 1) % chunk_steps == 0:
            files.append(_write_chunk(pending, out, first, last))
            pending = {c: [] for c in COLUMNS}
            first = None
            if progress is not None:
                progress(plan.step + 1, rows)
    if first is not None and pending["step"]:
        files.append(_write_chunk(pending, out, first, last))
    return {"until_step": until_step, "steps_walked": steps, "windows": windows, "rows": rows, "rows_per_source": per_source, "files": files,
            "position": view.stream_position()}


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
