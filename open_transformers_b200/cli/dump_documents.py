"""``pretrain-dump-documents``: detokenise the documents of a source's shards to Parquet (one row per document:
shard, index, length, text), several shards in parallel."""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import sys
from pathlib import Path


def _dump_one(job) -> int:
    prefix, tok_path, out, limit = job
    import pyarrow as pa
    import pyarrow.parquet as pq

    from ..data.indexed_dataset import IndexedDatasetReader
    from ..data.tokenizer import Tokenizer

    tok = Tokenizer(tok_path) if tok_path else None
    r = IndexedDatasetReader(prefix)
    rows = []
    for i in range(r.num_documents if limit is None else min(limit, r.num_documents)):
        ids = r.document(i)
        rows.append({"shard": Path(prefix).name, "doc_index": i, "length": int(len(ids)),
                     "text": tok.decode(ids) if tok else " ".join(str(int(t)) for t in ids)})
    pq.write_table(pa.Table.from_pylist(rows), out)
    return len(rows)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-dump-documents")
    ap.add_argument("--source-dir", required=True)
    ap.add_argument("--tokenizer")
    ap.add_argument("--out-dir", required=True)
    ap.add_argument("--limit", type=int)
    ap.add_argument("--workers", type=int, default=4)
    a = ap.parse_args(argv)
    from ..data.manifest import SourceManifest

    man = SourceManifest.load(Path(a.source_dir) / "manifest.yaml")
    Path(a.out_dir).mkdir(parents=True, exist_ok=True)
    jobs = [(str(Path(a.source_dir) / s.prefix), a.tokenizer, str(Path(a.out_dir) / (s.prefix + ".parquet")), a.limit) for s in man.shards]
    if a.workers > 1 and len(jobs) > 1:
        with mp.get_context("spawn").Pool(min(a.workers, len(jobs))) as pool:
            counts = pool.map(_dump_one, jobs)
    else:
        counts = [_dump_one(j) for j in jobs]
    print(json.dumps({"documents": sum(counts), "files": len(jobs)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
