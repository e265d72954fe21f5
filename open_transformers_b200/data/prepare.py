"""Corpus preparation: text iterators (parquet, jsonl, jsonl byte-segments for fan-out workers), sharding
into <= 1 GiB uint32 ``.bin/.idx`` shards with a manifest carrying per-shard blake2b digests, shard
inspection (reference src/pretrain/data/prepare.py:26-259)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Iterator

import numpy as np

from .indexed_dataset import IndexedDatasetReader, IndexedDatasetWriter
from .manifest import ShardInfo, SourceManifest, blake2b_file

SHARD_BYTES = 1 << 30


def iter_jsonl(path: str | Path, field: str = "text") -> Iterator[str]:
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                t = json.loads(line).get(field)
                if t:
                    yield t


def iter_jsonl_segment(path: str | Path, start: int, end: int, field: str = "text") -> Iterator[str]:
    """Lines whose FIRST byte lies in [start, end): workers given adjacent byte ranges of one file read every
    line exactly once."""
    with open(path, "rb") as f:
        if start > 0:
            f.seek(start - 1)
            if f.read(1) != b"\n":
                f.readline()       # finish the line that began before `start`
        while f.tell() < end:
            raw = f.readline()
            if not raw:
                break
            raw = raw.strip()
            if raw:
                t = json.loads(raw).get(field)
                if t:
                    yield t


def iter_parquet(path: str | Path, field: str = "text", batch_size: int = 1024) -> Iterator[str]:
    import pyarrow.parquet as pq

    pf = pq.ParquetFile(str(path))
    for batch in pf.iter_batches(batch_size=batch_size, columns=[field]):
        for t in batch.column(0).to_pylist():
            if t:
                yield t


def iter_texts(paths: Iterable[str | Path], field: str = "text") -> Iterator[str]:
    for p in paths:
        p = Path(p)
        yield from (iter_parquet(p, field) if p.suffix == ".parquet" else iter_jsonl(p, field))


def write_shards(texts: Iterable[str], tokenizer, out_dir: str | Path, name: str, shard_bytes: int = SHARD_BYTES, dtype=np.uint32,
                 batch_size: int = 512, raw_inputs: Iterable[str | Path] = (), filter_version: str = "") -> SourceManifest:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    item = np.dtype(dtype).itemsize
    shards: list[ShardInfo] = []
    writer, shard_id = None, 0

    def close():
        nonlocal writer, shard_id
        if writer is None:
            return
        prefix = "%s_%05d" % (name, shard_id)
        nd, nt = writer.num_documents, writer.token_count
        writer.finalize()
        shards.append(ShardInfo(prefix, nd, nt, blake2b_file(str(out / prefix) + ".bin"), blake2b_file(str(out / prefix) + ".idx")))
        writer = None
        shard_id += 1

    def add(ids):
        nonlocal writer
        if writer is not None and (writer.token_count + len(ids)) * item > shard_bytes and writer.num_documents > 0:
            close()
        if writer is None:
            writer = IndexedDatasetWriter(out / ("%s_%05d" % (name, shard_id)), dtype)
        writer.add_document(np.asarray(ids, dtype=np.int64))

    batch: list[str] = []
    for t in texts:
        batch.append(t)
        if len(batch) >= batch_size:
            for ids in tokenizer.encode_batch(batch):
                add(ids)
            batch = []
    if batch:
        for ids in tokenizer.encode_batch(batch):
            add(ids)
    close()
    man = SourceManifest(name=name, tokenizer_hash=getattr(tokenizer, "hash", ""), dtype=np.dtype(dtype).name, shards=shards,
                         filter_version=filter_version, raw_jsonl_blake2b={Path(p).name: blake2b_file(p) for p in raw_inputs})
    man.save(out / "manifest.yaml")
    return man


def merge_manifests(manifests: list[SourceManifest], name: str) -> SourceManifest:
    if len({m.tokenizer_hash for m in manifests}) > 1 or len({m.dtype for m in manifests}) > 1:
        raise ValueError("manifests disagree on tokenizer or dtype")
    raw = {}
    for m in manifests:
        raw.update(m.raw_jsonl_blake2b)
    return SourceManifest(name, manifests[0].tokenizer_hash, manifests[0].dtype, [s for m in manifests for s in m.shards],
                          manifests[0].filter_version, raw)


def inspect_shard(prefix: str | Path, tokenizer=None, n_docs: int = 3) -> dict:
    r = IndexedDatasetReader(prefix)
    lens = np.diff(r.doc_offsets)
    info = {"documents": r.num_documents, "tokens": r.token_count, "dtype": r.dtype.name,
            "doc_len_min": int(lens.min()) if len(lens) else 0, "doc_len_max": int(lens.max()) if len(lens) else 0,
            "doc_len_mean": float(lens.mean()) if len(lens) else 0.0, "samples": []}
    for i in range(min(n_docs, r.num_documents)):
        ids = r.document(i)[:64]
        info["samples"].append(tokenizer.decode(ids) if tokenizer is not None else [int(t) for t in ids])
    return info
