"""Step -> document map: for every optimizer step, micro-batch and window slot, which document pieces (source,
shard, document index, token range) make it up, and which data-parallel rank trained it. Written as Parquet;
built by walking the canonical stream by lengths only (reference src/pretrain/data/doc_map.py:28-198)."""
from __future__ import annotations

from pathlib import Path

from ..train.batch_schedule import owner_rank

COLUMNS = ["step", "microbatch", "slot", "dp_rank", "source", "shard", "doc_index", "doc_start", "length"]


def schema():
    import pyarrow as pa

    return pa.schema([("step", pa.int64()), ("microbatch", pa.int32()), ("slot", pa.int32()), ("dp_rank", pa.int32()), ("source", pa.string()),
                      ("shard", pa.int32()), ("doc_index", pa.int64()), ("doc_start", pa.int64()), ("length", pa.int64())])


def build_rows(view, n_steps: int, dp_world_size: int) -> list[dict]:
    rows = []
    for step, m, slot, source, shard, local, start, length in view.walk_doc_refs(n_steps):
        rows.append(dict(step=step, microbatch=m, slot=slot, dp_rank=owner_rank(m, world_size=dp_world_size), source=source, shard=shard,
                         doc_index=local, doc_start=start, length=length))
    return rows


def write_doc_map(view, n_steps: int, dp_world_size: int, out_path: str | Path) -> int:
    import pyarrow as pa
    import pyarrow.parquet as pq

    rows = build_rows(view, n_steps, dp_world_size)
    table = pa.Table.from_pylist(rows, schema=schema())
    Path(out_path).parent.mkdir(parents=True, exist_ok=True)
    pq.write_table(table, str(out_path))
    return len(rows)


def compare_position(view, expected_windows_emitted: int) -> bool:
    """True when the stream position reached by walking equals the position a checkpoint recorded."""
    return view.state().windows_emitted == expected_windows_emitted
