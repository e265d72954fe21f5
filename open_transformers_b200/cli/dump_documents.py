"""``pretrain-dump-documents``: the ``documents`` table of a corpus - every document of every shard detokenised to Parquet.

    pretrain-dump-documents --data-root data/shards --tokenizer tokenizer.json --out-dir DIR [--sources NAME ...]
                            [--workers N] [--batch-docs 2048] [--limit-shards N]

One file per shard, ``<out>/<source>/<shard id, 5 digits>_<prefix>.parquet``, rows ``source, shard_id, local_doc, n_tokens,
text`` - ``(source, shard_id, local_doc)`` is the document key of the step -> document map (``pretrain-dump-doc-map``). A file
that exists is skipped, so an interrupted run resumes; a file is renamed into place only when complete. Special tokens stay
in the text (a scraped document may contain the end-of-text marker literally; the text must match the stored ids).
(flags, file layout and columns: reference src/pretrain/cli/dump_documents.py:33-161)
"""
from __future__ import annotations

import argparse
import logging
import multiprocessing as mp
import sys
import time
from pathlib import Path

log = logging.getLogger("pretrain.dump_documents")
COLUMNS = ("source", "shard_id", "local_doc", "n_tokens", "text")
_tokenizer = None


def _worker_init(tokenizer_path: str) -> None:
    global _tokenizer
    from ..data.tokenizer import Tokenizer

    _tokenizer = Tokenizer(tokenizer_path)


def dump_shard(task) -> tuple[str, int, int, float]:
    """One shard -> one Parquet file. Returns (source, shard id, documents written or -1 when the file existed, seconds)."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    from ..data.indexed_dataset import IndexedDatasetReader

    source, shard_id, prefix, out_path, batch_docs = task
    out = Path(out_path)
    if out.exists():
        return source, shard_id, -1, 0.0
    t0 = time.time()
    reader = IndexedDatasetReader(prefix)
    sch = pa.schema([("source", pa.string()), ("shard_id", pa.int32()), ("local_doc", pa.int32()), ("n_tokens", pa.int32()), ("text", pa.large_string())])
    out.parent.mkdir(parents=True, exist_ok=True)
    part = out.with_suffix(".parquet.part")
    n = reader.num_documents
    with pq.ParquetWriter(part, sch, compression="zstd") as writer:
        for lo in range(0, n, batch_docs):
            hi = min(n, lo + batch_docs)
            ids = [reader.document(i).tolist() for i in range(lo, hi)]
            writer.write_table(pa.table({"source": pa.array([source] * (hi - lo), pa.string()), "shard_id": pa.array([shard_id] * (hi - lo), pa.int32()),
                                         "local_doc": pa.array(range(lo, hi), pa.int32()), "n_tokens": pa.array([len(x) for x in ids], pa.int32()),
                                         "text": pa.array(_tokenizer.decode_batch(ids, skip_special_tokens=False), pa.large_string())}, schema=sch))
    part.replace(out)
    return source, shard_id, n, time.time() - t0


def build_tasks(data_root: Path, out_dir: Path, sources, batch_docs: int, limit):
    """One task per shard of every ``<source>/manifest.yaml`` under ``data_root``. Output names carry the shard id (prefixes
    in different directories may share a base name); two shards that would land on one file are refused, because the
    skip-existing rule would silently drop one of them."""
    from ..data.manifest import SourceManifest

    tasks, taken = [], {}
    for mpath in sorted(data_root.glob("*/manifest.yaml")):
        man = SourceManifest.load(mpath)
        if sources and man.name not in sources:
            continue
        for sid, shard in enumerate(man.shards):
            if limit is not None and sid >= limit:
                break
            stem = Path(shard.prefix)
            prefix = stem if stem.is_absolute() else mpath.parent / stem
            out = out_dir / man.name / ("%05d_%s.parquet" % (sid, stem.name))
            if str(out) in taken:
                raise ValueError("duplicate output %s for shards %s and %s" % (out, taken[str(out)], prefix))
            taken[str(out)] = str(prefix)
            tasks.append((man.name, sid, str(prefix), str(out), batch_docs))
    return tasks


def run(a) -> int:
    tasks = build_tasks(Path(a.data_root), Path(a.out_dir), a.sources, a.batch_docs, a.limit_shards)
    if not tasks:
        log.error("no shards found under %s", a.data_root)
        return 1
    log.info("%d shards, %d workers, out=%s", len(tasks), a.workers, a.out_dir)
    t0 = time.time()
    written = skipped = docs = 0

    def account(result):
        nonlocal written, skipped, docs
        source, sid, n, dt = result
        if n < 0:
            skipped += 1
            return
        written += 1
        docs += n
        if written % 10 == 0 or dt > 300:
            log.info("%d/%d shards (%d skipped), %d docs, last %s/%d %.0fs, elapsed %.0fs", written + skipped, len(tasks), skipped, docs, source, sid,
                     dt, time.time() - t0)

    if a.workers > 1 and len(tasks) > 1:
        with mp.get_context("spawn").Pool(min(a.workers, len(tasks)), initializer=_worker_init, initargs=(a.tokenizer,)) as pool:
            for result in pool.imap_unordered(dump_shard, tasks):
                account(result)
    else:
        _worker_init(a.tokenizer)
        for task in tasks:
            account(dump_shard(task))
    log.info("finished: %d written, %d skipped, %d docs, %.0fs", written, skipped, docs, time.time() - t0)
    return 0


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    ap = argparse.ArgumentParser(prog="pretrain-dump-documents")
    ap.add_argument("--data-root", required=True, help="directory holding <source>/manifest.yaml and the shards")
    ap.add_argument("--tokenizer", required=True, help="tokenizer.json the shards were prepared with")
    ap.add_argument("--out-dir", required=True, help="output root; files land at <out>/<source>/<shard id>_<prefix>.parquet")
    ap.add_argument("--sources", nargs="*", default=None, help="subset of source names (default: all)")
    ap.add_argument("--workers", type=int, default=max(1, mp.cpu_count() - 2))
    ap.add_argument("--batch-docs", type=int, default=2048, help="documents decoded per batch / row group")
    ap.add_argument("--limit-shards", type=int, default=None, help="debugging: only the first N shards per source")
    return run(ap.parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
