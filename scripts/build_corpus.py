#!/usr/bin/env python
"""Corpus assembly helpers: a two-pass bucket shuffle of a JSONL file too large for memory, and a fan-out plan
that splits one JSONL into byte segments for parallel sharding workers (each worker then runs
`pretrain-prepare-data shard --segment start:end`)."""
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


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("shuffle"); s.add_argument("src"); s.add_argument("dst"); s.add_argument("--seed", type=int, default=0)
    s.add_argument("--buckets", type=int, default=64)
    p = sub.add_parser("plan"); p.add_argument("src"); p.add_argument("--workers", type=int, default=8)
    a = ap.parse_args()
    if a.cmd == "shuffle":
        print(json.dumps({"lines": shuffle_jsonl(a.src, a.dst, a.seed, a.buckets)}))
    else:
        print(json.dumps(segment_plan(a.src, a.workers), indent=1))


if __name__ == "__main__":
    main()
