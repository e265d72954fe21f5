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
                 batch_size: int = 512, raw_inputs: Iterable[str | Path] = (), filter_version: str = "", prefix_tag: str = "",
                 manifest_name: str = "manifest.yaml") -> SourceManifest:
    """``prefix_tag`` (e.g. ``_w03``) goes between the source name and the shard number and ``manifest_name`` names the
    manifest file: fan-out workers write side by side into one directory and ``merge_worker_manifests`` joins them."""
    out = Path(out_dir)
    name_tag = name + prefix_tag
    out.mkdir(parents=True, exist_ok=True)
    item = np.dtype(dtype).itemsize
    shards: list[ShardInfo] = []
    writer, shard_id = None, 0

    def close():
        nonlocal writer, shard_id
        if writer is None:
            return
        prefix = "%s_%05d" % (name_tag, shard_id)
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
            writer = IndexedDatasetWriter(out / ("%s_%05d" % (name_tag, shard_id)), dtype)
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
    man.save(out / manifest_name)
    return man


def iter_jsonl_worker_share(paths: Iterable[str | Path], worker_id: int, num_workers: int, field: str = "text") -> Iterator[str]:
    """Worker ``worker_id`` of ``num_workers``: its byte range of every file (lines are whole; every line is read by exactly
    one worker)."""
    for p in paths:
        size = Path(p).stat().st_size
        yield from iter_jsonl_segment(p, size * worker_id // num_workers, size * (worker_id + 1) // num_workers, field)


def merge_worker_manifests(out_dir: str | Path, expected_workers: int = 0, remove: bool = False) -> SourceManifest:
    """Join the ``manifest.w*.yaml`` files fan-out workers left in ``out_dir`` into ``manifest.yaml``: shard lists in
    worker order (so the order on disk is reproducible), raw-input digests united (the same file with two different
    digests is an error), name / tokenizer / dtype required to agree. (reference src/pretrain/cli/prepare_data.py:140-210)"""
    out = Path(out_dir)
    parts = sorted(out.glob("manifest.w*.yaml"))
    if not parts:
        raise ValueError("no manifest.w*.yaml under %s - did the fan-out workers run?" % out)
    if expected_workers and len(parts) != expected_workers:
        raise ValueError("expected %d per-worker manifests under %s, found %d: %s" % (expected_workers, out, len(parts), [p.name for p in parts]))
    mans = [SourceManifest.load(p) for p in parts]
    first = mans[0]
    raw: dict[str, str] = {}
    for p, m in zip(parts, mans):
        for what in ("name", "tokenizer_hash", "dtype"):
            if getattr(m, what) != getattr(first, what):
                raise ValueError("%s mismatch in %s: %s vs %s" % (what, p, getattr(m, what), getattr(first, what)))
        for fname, digest in m.raw_jsonl_blake2b.items():
            if raw.setdefault(fname, digest) != digest:
                raise ValueError("raw_jsonl_blake2b conflict for %r in %s: %s vs %s" % (fname, p, digest, raw[fname]))
    merged = SourceManifest(first.name, first.tokenizer_hash, first.dtype, [s for m in mans for s in m.shards], first.filter_version, raw)
    merged.save(out / "manifest.yaml")
    if remove:
        for p in parts:
            p.unlink()
    return merged


def bytes_per_token(tokenizer, text: str) -> float:
    return len(text.encode("utf-8")) / max(len(tokenizer.encode(text)), 1)


def write_random_sources(out_dir: str | Path, docs_a: int = 2000, docs_b: int = 1000, min_doc_len: int = 64, max_doc_len: int = 512,
                         vocab_size: int = 128_256, seed: int = 0) -> list[SourceManifest]:
    """Two sources of random documents, ``synth_a`` and ``synth_b`` (the pair ``configs/data/synthetic.yaml`` names), one
    shard each, no tokenizer involved: token ids uniform in [1, vocab_size), lengths uniform in [min, max]."""
    out = Path(out_dir)
    rng = np.random.default_rng(seed)
    made = []
    for name, n_docs in (("synth_a", docs_a), ("synth_b", docs_b)):
        d = out / name
        d.mkdir(parents=True, exist_ok=True)
        prefix = "%s_00000" % name
        with IndexedDatasetWriter(d / prefix, np.uint32) as w:
            for _ in range(n_docs):
                w.add_document(rng.integers(1, vocab_size, size=int(rng.integers(min_doc_len, max_doc_len + 1)), dtype=np.uint32))
        man = SourceManifest(name, "synthetic-no-tokenizer", "uint32", [ShardInfo(prefix, n_docs, IndexedDatasetReader(d / prefix).token_count)])
        man.save(d / "manifest.yaml")
        made.append(man)
    return made


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
