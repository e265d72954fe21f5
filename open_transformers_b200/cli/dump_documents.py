"""``pretrain-dump-documents``: a prepared corpus turned back into text, one Parquet file per shard.

    pretrain-dump-documents --data-root data/shards --tokenizer tokenizer.json --out-dir DIR [--sources NAME ...]
                            [--workers N] [--batch-docs 2048] [--limit-shards N]

Layout: ``<out>/<source>/<five-digit shard id>_<shard prefix>.parquet`` with the columns ``source, shard_id, local_doc,
n_tokens, text``. The first three are the document key that ``pretrain-dump-doc-map`` writes, so "which text did step 812
read" is a join of the two tables. Decoding keeps special tokens: web text now and then contains the end-of-text marker as
literal characters, the tokenizer stored it as the special id, and the text has to correspond to the ``n_tokens`` ids on
disk. Work is split by shard over a process pool; a shard whose file exists is left alone (the job can be re-run after an
interruption), and a file appears under its final name only once it is whole.
(flag set, file naming and columns: reference src/pretrain/cli/dump_documents.py:33-107)
"""
from __future__ import annotations

import argparse
import dataclasses
import logging
import multiprocessing as mp
import sys
import time
from pathlib import Path

log = logging.getLogger("pretrain.dump_documents")
COLUMNS = ("source", "shard_id", "local_doc", "n_tokens", "text")
SKIPPED = -1
_decoder = None   # per-process tokenizer, set by the pool initializer


@dataclasses.dataclass(frozen=True)
class ShardJob:
    source: str
    shard_id: int
    prefix: str          # <dir>/<name> of the .bin / .idx pair
    target: str          # Parquet file to produce
    batch_docs: int


def _load_decoder(tokenizer_path: str) -> None:
    global _decoder
    from ..data.tokenizer import Tokenizer

    _decoder = Tokenizer(tokenizer_path)


def _schema():
    import pyarrow as pa

    kinds = {"source": pa.string(), "shard_id": pa.int32(), "local_doc": pa.int32(), "n_tokens": pa.int32(), "text": pa.large_string()}
    return pa.schema([(c, kinds[c]) for c in COLUMNS])


def _row_groups(job: ShardJob, schema):
    """Tables of at most ``batch_docs`` documents, in document order."""
    import pyarrow as pa

    from ..data.indexed_dataset import IndexedDatasetReader

    shard = IndexedDatasetReader(job.prefix)
    for first in range(0, len(shard), job.batch_docs):
        docs = range(first, min(len(shard), first + job.batch_docs))
        ids = [shard.document(d).tolist() for d in docs]
        cols = {"source": [job.source] * len(ids), "shard_id": [job.shard_id] * len(ids), "local_doc": list(docs),
                "n_tokens": [len(t) for t in ids], "text": _decoder.decode_batch(ids, skip_special_tokens=False)}
        yield pa.table({c: pa.array(cols[c], schema.field(c).type) for c in COLUMNS}, schema=schema)


def dump_shard(job) -> tuple[str, int, int, float]:
    """Write one shard's file; ``(source, shard id, documents written, seconds)``, with ``SKIPPED`` documents when the file
    was already there. Accepts a ``ShardJob`` or its fields as a tuple."""
    import pyarrow.parquet as pq

    job = job if isinstance(job, ShardJob) else ShardJob(*job)
    final = Path(job.target)
    if final.exists():
        return job.source, job.shard_id, SKIPPED, 0.0
    began, written = time.time(), 0
    final.parent.mkdir(parents=True, exist_ok=True)
    unfinished = final.with_suffix(".parquet.part")
    schema = _schema()
    with pq.ParquetWriter(unfinished, schema, compression="zstd") as sink:
        for table in _row_groups(job, schema):
            sink.write_table(table)
            written += table.num_rows
    unfinished.replace(final)
    return job.source, job.shard_id, written, time.time() - began


def build_tasks(data_root: Path, out_dir: Path, sources, batch_docs: int, limit) -> list[ShardJob]:
    """Every shard of every ``<source>/manifest.yaml`` below ``data_root`` (restricted to ``sources`` and to the first
    ``limit`` shards of each, when given). The shard id is part of the file name because prefixes that live in different
    directories can share their last component; if two shards still map to one file - two manifests carrying one source
    name - that is an error, since "skip what exists" would quietly lose one of them."""
    from ..data.manifest import SourceManifest

    jobs, owner_of = [], {}
    for manifest_file in sorted(data_root.glob("*/manifest.yaml")):
        manifest = SourceManifest.load(manifest_file)
        if sources and manifest.name not in sources:
            continue
        shards = manifest.shards if limit is None else manifest.shards[:limit]
        for shard_id, shard in enumerate(shards):
            rel = Path(shard.prefix)
            prefix = str(rel if rel.is_absolute() else manifest_file.parent / rel)
            target = str(out_dir / manifest.name / ("%05d_%s.parquet" % (shard_id, rel.name)))
            if target in owner_of:
                raise ValueError("duplicate output %s: both %s and %s would be written there" % (target, owner_of[target], prefix))
            owner_of[target] = prefix
            jobs.append(ShardJob(manifest.name, shard_id, prefix, target, batch_docs))
    return jobs


class _Tally:
    def __init__(self, total: int):
        self.total, self.written, self.skipped, self.docs, self.began = total, 0, 0, 0, time.time()

    def add(self, outcome) -> None:
        source, shard_id, n, seconds = outcome
        if n == SKIPPED:
            self.skipped += 1
            return
        self.written += 1
        self.docs += n
        if self.written % 10 == 0 or seconds > 300:
            log.info("%d of %d shards done (%d already present), %d documents; %s shard %d took %.0fs; %.0fs so far", self.written + self.skipped,
                     self.total, self.skipped, self.docs, source, shard_id, seconds, time.time() - self.began)


def run(a) -> int:
    jobs = build_tasks(Path(a.data_root), Path(a.out_dir), a.sources, a.batch_docs, a.limit_shards)
    if not jobs:
        log.error("no shards found under %s", a.data_root)
        return 1
    procs = max(1, min(a.workers, len(jobs)))
    log.info("%d shards to decode with %d process(es) into %s", len(jobs), procs, a.out_dir)
    tally = _Tally(len(jobs))
    if procs == 1:
        _load_decoder(a.tokenizer)
        for job in jobs:
            tally.add(dump_shard(job))
    else:
        with mp.get_context("spawn").Pool(procs, initializer=_load_decoder, initargs=(a.tokenizer,)) as pool:
            for outcome in pool.imap_unordered(dump_shard, jobs):
                tally.add(outcome)
    log.info("finished: %d written, %d skipped, %d docs, %.0fs", tally.written, tally.skipped, tally.docs, time.time() - tally.began)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pretrain-dump-documents", description="Detokenise the shards of a prepared corpus into Parquet.")
    ap.add_argument("--data-root", required=True, help="parent directory of the sources (each with its manifest.yaml and shards)")
    ap.add_argument("--tokenizer", required=True, help="the tokenizer.json that produced the shards")
    ap.add_argument("--out-dir", required=True, help="root of the output tree: <out>/<source>/<shard id>_<prefix>.parquet")
    ap.add_argument("--sources", nargs="*", default=None, help="only these source names")
    ap.add_argument("--workers", type=int, default=max(1, mp.cpu_count() - 2), help="decoder processes")
    ap.add_argument("--batch-docs", type=int, default=2048, help="documents per decode call and per Parquet row group")
    ap.add_argument("--limit-shards", type=int, default=None, help="stop after this many shards of each source (for trying things out)")
    return ap


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
