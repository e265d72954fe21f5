#!/usr/bin/env python
"""Corpus assembly: the local half of the reference's scripts/build_corpus.py.

  shuffle SRC DST [--seed --buckets]            two-pass bucket shuffle of a JSONL file too large for memory
  plan SRC [--workers]                          byte segments of one JSONL for parallel sharding workers
  shard SRC --tokenizer T --out-dir D --name N [--workers W] [--shard-bytes B]
                                                fan-out: W worker processes tokenise one byte segment each into
                                                <D>/w<k>/ and the worker manifests are merged, in worker order, into
                                                <D>/manifest.yaml (shard prefixes become w<k>/<name>_<id>)
  pull SOURCE                                   the reference's dataset pullers (DCLM, FineWeb, proof-pile, Dolma 3 mix,
                                                the Stack via Software Heritage) need network access to their hosts;
                                                this build has none, so the subcommand names the source and exits 2

A segment boundary falls on a line boundary (a worker starts at the first line that begins inside its segment), so the
union of the workers' documents is the file's documents, each exactly once, in file order across workers.
"""
import argparse
import hashlib
import json
import os
import random
import sys
import tempfile
from pathlib import Path


def shuffle_jsonl(src, dst, seed=0, n_buckets=64, tmp_dir=None):
    """Pass 1 scatters lines into `n_buckets` files by a seeded hash of (seed, line number); pass 2 shuffles each
    bucket in memory with a seeded RNG and concatenates them. Deterministic in (seed, n_buckets)."""
    tmp = Path(tempfile.mkdtemp(dir=tmp_dir))
    files = [open(tmp / ("b%04d" % i), "wb") for i in range(n_buckets)]
    with open(src, "rb") as f:
        for i, line in enumerate(f):
            if not line.strip():
                continue
            h = hashlib.blake2b(b"%d:%d" % (seed, i), digest_size=8).digest()
            files[int.from_bytes(h, "big") % n_buckets].write(line if line.endswith(b"\n") else line + b"\n")
    for fh in files:
        fh.close()
    n = 0
    with open(dst, "wb") as out:
        for i in range(n_buckets):
            p = tmp / ("b%04d" % i)
            lines = p.read_bytes().splitlines(keepends=True)
            random.Random(seed * 1_000_003 + i).shuffle(lines)
            out.writelines(lines)
            n += len(lines)
            p.unlink()
    tmp.rmdir()
    return n


def segment_plan(path, workers):
    size = os.path.getsize(path)
    cuts = [size * i // workers for i in range(workers + 1)]
    return [{"worker": i, "segment": "%d:%d" % (cuts[i], cuts[i + 1])} for i in range(workers)]


def _shard_worker(args):
    """One fan-out worker: tokenise the JSONL lines that begin inside [start, end) into its own directory."""
    src, start, end, tokenizer_path, out_dir, name, shard_bytes, field = args
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from open_transformers_b200.data.prepare import iter_jsonl_segment, write_shards
    from open_transformers_b200.data.tokenizer import Tokenizer

    man = write_shards(iter_jsonl_segment(src, start, end, field), Tokenizer(tokenizer_path), out_dir, name, shard_bytes=shard_bytes)
    return str(Path(out_dir) / "manifest.yaml"), man.total_documents, man.total_tokens


def shard_source(src, tokenizer_path, out_dir, name, workers=8, shard_bytes=1 << 30, field="text"):
    """Parallel sharding of one JSONL file; returns the merged manifest (also written to <out_dir>/manifest.yaml)."""
    import multiprocessing as mp

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from open_transformers_b200.data.manifest import ShardInfo, SourceManifest, blake2b_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    jobs = []
    for seg in segment_plan(src, workers):
        a, b = (int(x) for x in seg["segment"].split(":"))
        jobs.append((str(src), a, b, str(tokenizer_path), str(out / ("w%03d" % seg["worker"])), name, shard_bytes, field))
    with mp.get_context("spawn").Pool(min(workers, os.cpu_count() or 1)) as pool:
        results = pool.map(_shard_worker, jobs)
    shards, first = [], None
    for k, (mpath, _nd, _nt) in enumerate(results):
        man = SourceManifest.load(mpath)
        first = first or man
        for sh in man.shards:  # worker order, then shard order: the merged manifest lists documents in file order
            shards.append(ShardInfo("w%03d/%s" % (k, sh.prefix), sh.num_documents, sh.token_count, sh.bin_blake2b, sh.idx_blake2b))
    merged = SourceManifest(name=name, tokenizer_hash=first.tokenizer_hash, dtype=first.dtype, shards=shards,
                            raw_jsonl_blake2b={Path(src).name: blake2b_file(str(src))})
    merged.save(out / "manifest.yaml")
    return merged


PULL_SOURCES = {"dclm": "mlfoundations/dclm-baseline-1.0 (HF hub)", "fineweb": "HuggingFaceFW/fineweb-edu (HF hub)",
                "proof": "proof-pile-2 subsets (HF hub)", "dolma3_dolmino_mix": "allenai/dolma3 + dolmino mix (HF hub)",
                "stack": "Software Heritage S3 blobs listed by the-stack-v2"}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("shuffle"); s.add_argument("src"); s.add_argument("dst"); s.add_argument("--seed", type=int, default=0)
    s.add_argument("--buckets", type=int, default=64)
    p = sub.add_parser("plan"); p.add_argument("src"); p.add_argument("--workers", type=int, default=8)
    h = sub.add_parser("shard"); h.add_argument("src"); h.add_argument("--tokenizer", required=True); h.add_argument("--out-dir", required=True)
    h.add_argument("--name", required=True); h.add_argument("--workers", type=int, default=8); h.add_argument("--shard-bytes", type=int, default=1 << 30)
    h.add_argument("--field", default="text")
    q = sub.add_parser("pull"); q.add_argument("source", choices=sorted(PULL_SOURCES)); q.add_argument("--docs", type=int, default=0)
    a = ap.parse_args()
    if a.cmd == "shuffle":
        print(json.dumps({"lines": shuffle_jsonl(a.src, a.dst, a.seed, a.buckets)}))
    elif a.cmd == "plan":
        print(json.dumps(segment_plan(a.src, a.workers), indent=1))
    elif a.cmd == "shard":
        m = shard_source(a.src, a.tokenizer, a.out_dir, a.name, a.workers, a.shard_bytes, a.field)
        print(json.dumps({"shards": len(m.shards), "documents": m.total_documents, "tokens": m.total_tokens}))
    else:
        print("pull %s: needs network access to %s; bring the JSONL files in by other means and continue with "
              "`shuffle` and `shard`" % (a.source, PULL_SOURCES[a.source]), file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
