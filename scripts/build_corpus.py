#!/usr/bin/env python
"""Corpus assembly: the local half of the reference's scripts/build_corpus.py.

  shuffle SRC DST [--seed --buckets]            two-pass bucket shuffle of a JSONL file too large for memory
  plan SRC [--workers]                          byte segments of one JSONL for parallel sharding workers
  shard SRC --tokenizer T --out-dir D --name N [--workers W] [--shard-bytes B]
                                                fan-out: W worker processes tokenise one byte segment each into
                                                <D>/w<k>/ and the worker manifests are merged, in worker order, into
                                                <D>/manifest.yaml (shard prefixes become w<k>/<name>_<id>)
  pull SOURCE --docs N --raw-dir D              resumable streaming pull of one source into <D>/<source>.jsonl: DCLM-Baseline,
                                                FineWeb-Edu (int_score >= 3), Proof-Pile-2 (three configurations by weight),
                                                the Dolma 3 / Dolmino mix (round-robin over its source directories) and the
                                                Stack v2 (file contents fetched from Software Heritage). Needs the `datasets`
                                                / `huggingface_hub` / `boto3` packages and network access to their hosts.
  build [--preset P | --docs-<source> N ...]    pull -> shuffle -> shard for every source of the plan; each stage is skipped
                                                when its output (manifest, `.shuffled` mark) is already there

Resume: a pull appends to its JSONL. On entry the file is cut back to its last complete, valid line on a 1000-document
boundary, and a `<file>.scanned` note holds how many raw rows of the stream had been consumed at that boundary, so a restart
skips exactly those rows even where a filter drops most of them. `<file>.revision` records the dataset commit that was read.

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


def shard_source(src, tokenizer_path, out_dir, name, workers=8, shard_bytes=1 << 30, field="text", prefix_tag="", manifest_name="manifest.yaml"):
    """Parallel sharding of one JSONL file; returns the merged manifest (also written to <out_dir>/<manifest_name>).
    ``prefix_tag`` (e.g. ``_w03``: one machine of a fan-out) keeps this call's shard directories apart from its siblings'."""
    import multiprocessing as mp

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from open_transformers_b200.data.manifest import ShardInfo, SourceManifest, blake2b_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    jobs = []
    sub = prefix_tag.strip("_") + "/" if prefix_tag else ""
    for seg in segment_plan(src, workers):
        a, b = (int(x) for x in seg["segment"].split(":"))
        jobs.append((str(src), a, b, str(tokenizer_path), str(out / (sub + "w%03d" % seg["worker"])), name, shard_bytes, field))
    with mp.get_context("spawn").Pool(min(workers, os.cpu_count() or 1)) as pool:
        results = pool.map(_shard_worker, jobs)
    shards, first = [], None
    for k, (mpath, _nd, _nt) in enumerate(results):
        man = SourceManifest.load(mpath)
        first = first or man
        for sh in man.shards:  # worker order, then shard order: the merged manifest lists documents in file order
            shards.append(ShardInfo("%sw%03d/%s" % (sub, k, sh.prefix), sh.num_documents, sh.token_count, sh.bin_blake2b, sh.idx_blake2b))
    merged = SourceManifest(name=name, tokenizer_hash=first.tokenizer_hash, dtype=first.dtype, shards=shards,
                            raw_jsonl_blake2b={Path(src).name: blake2b_file(str(src))})
    merged.save(out / manifest_name)
    return merged


# ------------------------------------------------------------------------------------------------ resumable pulls
RESUME_CHUNK = 1000
PRESETS = {"100m_proxy": {"dclm": 300_000, "fineweb": 70_000, "stack": 200_000, "proof": 15_000},
           "1b_proxy": {"dclm": 6_000_000, "fineweb": 1_400_000, "stack": 4_000_000, "proof": 300_000}}
PROOF_WEIGHTS = {"arxiv": 0.5, "open-web-math": 0.3, "algebraic-stack": 0.2}
PERMISSIVE = {"mit", "apache-2.0", "bsd-2-clause", "bsd-3-clause", "isc", "unlicense", "cc0-1.0", "0bsd", "zlib", "bsl-1.0"}


def _note(out, kind):
    return Path(str(out) + "." + kind)


def count_valid_lines(out):
    """(complete parseable lines from the start of `out`, byte offset after each of them)."""
    ends, pos = [], 0
    if Path(out).is_file():
        with open(out, "rb") as f:
            for line in f:
                if not line.endswith(b"\n"):
                    break
                try:
                    json.loads(line)
                except ValueError:
                    break
                pos += len(line)
                ends.append(pos)
    return len(ends), ends


def read_cursor(out):
    try:
        return json.loads(_note(out, "scanned").read_text())
    except (OSError, ValueError):
        return {}


def write_cursor(out, cursor):
    tmp = _note(out, "scanned.tmp")
    tmp.write_text(json.dumps(cursor))
    os.replace(tmp, _note(out, "scanned"))


def resume_point(out, log=None):
    """Bring `out` and its `.scanned` note into agreement and return (documents kept, rows scanned per stream, documents
    taken per stream). The note is written after the file was flushed, at every 1000th document and at the end of a pull, so
    the file holds at least the documents the note accounts for: anything beyond them (written after the last note, or a
    torn last line) is cut off. A file without a note starts over."""
    out = Path(out)
    n_valid, ends = count_valid_lines(out)
    cursor = read_cursor(out)
    taken = {k: int(v) for k, v in cursor.get("taken", {}).items()}
    scanned = {k: int(v) for k, v in cursor.get("scanned", {}).items()}
    keep = sum(taken.values())
    if keep > n_valid:
        raise RuntimeError("%s holds %d valid documents but its .scanned note accounts for %d: the file was damaged; remove both to start over"
                           % (out, n_valid, keep))
    if out.is_file() and (keep < n_valid or (ends[-1] if ends else 0) != out.stat().st_size):
        if log:
            log("%s: keeping %d of %d documents (the rest was written after the last resume note)" % (out.name, keep, n_valid))
        with open(out, "rb+") as f:
            f.truncate(ends[keep - 1] if keep else 0)
    return keep, scanned, taken


class Stream:
    """One stream of raw rows with a filter: `rows(skip)` yields the stream's rows after the first `skip`; `keep(row)`
    returns the document text or None."""

    def __init__(self, key, rows, keep):
        self.key, self.rows, self.keep = key, rows, keep


def pull(out, target, streams, chunk=RESUME_CHUNK, log=None):
    """Append documents from `streams` - [(Stream, quota)], in order; quota None = whatever is still missing - until `out`
    holds `target` documents or the streams end. Returns (documents in the file, rows scanned per stream)."""
    out = Path(out)
    out.parent.mkdir(parents=True, exist_ok=True)
    have, scanned, taken = resume_point(out, log)
    with open(out, "a", encoding="utf-8") as f:
        for stream, quota in streams:
            n_scanned, n_taken = scanned.get(stream.key, 0), taken.get(stream.key, 0)
            want = (target - have) if quota is None else min(quota - n_taken, target - have)
            if want <= 0:
                continue
            for row in stream.rows(n_scanned):
                n_scanned += 1
                text = stream.keep(row)
                if not text:
                    continue
                f.write(json.dumps({"text": text}) + "\n")
                have, n_taken, want = have + 1, n_taken + 1, want - 1
                if have % chunk == 0:
                    f.flush()
                    scanned[stream.key], taken[stream.key] = n_scanned, n_taken
                    write_cursor(out, {"scanned": scanned, "taken": taken})
                    if log:
                        log("%s: %d documents, %d rows of %s scanned" % (out.name, have, n_scanned, stream.key))
                if want <= 0:
                    break
            scanned[stream.key], taken[stream.key] = n_scanned, n_taken
        f.flush()
    write_cursor(out, {"scanned": scanned, "taken": taken})
    return have, scanned


def split_by_weight(total, weights):
    """Integer shares of `total` in proportion to `weights`; the last key absorbs the rounding."""
    keys, norm = list(weights), sum(weights.values())
    shares = {k: int(total * weights[k] / norm) for k in keys[:-1]}
    shares[keys[-1]] = total - sum(shares.values())
    return shares


def hub_rows(repo, revision="main", name=None, split="train", data_files=None):
    """`rows(skip)` over a Hugging Face dataset in streaming mode (imports `datasets` on first use)."""
    def rows(skip):
        from datasets import load_dataset

        ds = load_dataset(repo, name=name, split=split, streaming=True, revision=revision, data_files=data_files)
        return iter(ds.skip(skip) if skip else ds)
    return rows


def text_of(row):
    t = row.get("text")
    return t if isinstance(t, str) and t.strip() else None


def is_eval_split(path):
    """Files of a dataset repository that hold evaluation or held-out data and must not enter a training pull."""
    low = path.lower()
    return any(part in low for part in ("/test", "/valid", "/eval", "/dev/", "heldout", "held_out", "-test-", "-validation-"))


def round_robin_files(files_by_source):
    """One file per source per round, sources in name order, until every source is exhausted: a partial pull samples all
    sources evenly instead of finishing whichever sorts first."""
    queues = {k: list(v) for k, v in sorted(files_by_source.items())}
    while any(queues.values()):
        for k in list(queues):
            if queues[k]:
                yield k, queues[k].pop(0)


def ordered_fetch(items, fetch, workers=64, window=None):
    """`fetch(item)` for every item with up to `workers` in flight, results yielded in input order (None results kept)."""
    from collections import deque
    from concurrent.futures import ThreadPoolExecutor

    window = window or 4 * workers
    with ThreadPoolExecutor(max_workers=workers) as ex:
        pending = deque()
        for item in items:
            pending.append((item, ex.submit(fetch, item)))
            if len(pending) >= window:
                it, fut = pending.popleft()
                yield it, fut.result()
        while pending:
            it, fut = pending.popleft()
            yield it, fut.result()


def swh_fetcher():
    """`fetch(row)` -> decoded file content from the Software Heritage bucket (anonymous S3), or None."""
    import gzip

    import boto3
    from botocore import UNSIGNED
    from botocore.config import Config

    s3 = boto3.client("s3", config=Config(signature_version=UNSIGNED, max_pool_connections=128))

    def fetch(row):
        try:
            body = s3.get_object(Bucket="softwareheritage", Key="content/" + row["blob_id"])["Body"].read()
            return gzip.decompress(body).decode(row.get("src_encoding") or "utf-8", errors="strict")
        except Exception:
            return None
    return fetch


def source_streams(source, target, fetch_blob=None, list_files=None, workers=64, worker_id=0, num_workers=1):
    """[(Stream, quota)] of one named source. `fetch_blob` / `list_files` stand in for the network in tests. ``num_workers`` > 1
    (the Stack): this process takes every ``num_workers``-th metadata row starting at ``worker_id``."""
    if source == "dclm":
        return [(Stream("dclm", hub_rows("mlfoundations/dclm-baseline-1.0"), text_of), None)]
    if source == "fineweb":
        return [(Stream("fineweb", hub_rows("HuggingFaceFW/fineweb-edu"), lambda r: text_of(r) if r.get("int_score", 0) >= 3 else None), None)]
    if source == "proof":
        shares = split_by_weight(target, PROOF_WEIGHTS)
        return [(Stream("proof/" + cfg, hub_rows("EleutherAI/proof-pile-2", name=cfg), text_of), shares[cfg]) for cfg in PROOF_WEIGHTS]
    if source == "dolma3_dolmino_mix":
        repo = "allenai/dolma3_dolmino_mix-100B-1125"
        if list_files is None:
            from huggingface_hub import HfApi

            list_files = lambda: HfApi().list_repo_files(repo, repo_type="dataset")  # noqa: E731
        by_source = {}
        for path in sorted(list_files()):
            if path.endswith((".jsonl", ".jsonl.gz", ".jsonl.zst", ".json.gz", ".parquet")) and not is_eval_split("/" + path):
                by_source.setdefault(path.split("/")[1] if path.count("/") >= 2 else path.split("/")[0], []).append(path)
        order = [path for _src, path in round_robin_files(by_source)]

        def rows(skip):
            seen = 0
            for path in order:
                for row in hub_rows(repo, data_files=path)(0):
                    seen += 1
                    if seen > skip:
                        yield row
        return [(Stream("dolma3", rows, text_of), None)]
    if source == "stack":
        fetch = fetch_blob or swh_fetcher()
        meta = hub_rows("bigcode/the-stack-v2-dedup")

        def rows(skip):
            permissive = (r for i, r in enumerate(meta(skip)) if num_workers <= 1 or (skip + i) % num_workers == worker_id)
            for row, content in ordered_fetch(permissive, lambda r: fetch(r) if (r.get("detected_licenses") and set(map(str.lower, r["detected_licenses"])) <= PERMISSIVE) else None, workers):
                yield {"text": content}
        return [(Stream("stack", rows, text_of), None)]
    raise ValueError("unknown source %r" % source)


PULL_SOURCES = ("dclm", "fineweb", "stack", "proof", "dolma3_dolmino_mix")
# the names the data recipes use for these sources (configs/data/*.yaml: manifest name and shard directory)
CORPUS_NAME = {"dclm": "dclm_baseline", "fineweb": "fineweb_edu", "stack": "stack_v2_permissive", "proof": "proof_pile_2",
               "dolma3_dolmino_mix": "dolma3_dolmino_mix"}
SHORT_NAME = {v: k for k, v in CORPUS_NAME.items()}
MIDTRAIN_SOURCES = ("dolma3_dolmino_mix",)   # built only when named with --only


def build(counts, raw_dir, shard_dir, tokenizer, suffix="_proxy", shuffle_seed=0, workers=8, delete_raw=False, only=None, pull_fn=None, log=print,
          concurrency=None, worker_id=0, num_workers=1):
    """pull -> shuffle -> shard per source; every stage is idempotent (manifest present: source done; `.shuffled` note: shuffle
    done). Files carry the recipes' source names (``dclm`` -> ``<shard_dir>/dclm_baseline<suffix>``, manifest name
    ``dclm_baseline``). ``concurrency``: {source: parallel fetches}. ``num_workers`` > 1 (the Stack only): this process is worker
    ``worker_id`` of a fan-out over several machines - it pulls its slice into ``<name>_w<K>.jsonl`` and writes ``<name>_w<K>_*``
    shards with ``manifest.w<K>.yaml``; ``pretrain-prepare-data merge-manifests --output-dir`` joins them afterwards.
    Returns {source: manifest path}."""
    raw_dir, shard_dir = Path(raw_dir), Path(shard_dir)
    only = [SHORT_NAME.get(x, x) for x in only] if only else None
    concurrency = concurrency or {}
    fan_out = num_workers > 1
    if fan_out and only != ["stack"]:
        raise ValueError("--num-workers > 1 is only supported with --only stack_v2_permissive")
    done = {}
    for source, n in counts.items():
        if (only and source not in only) or n <= 0 or (source in MIDTRAIN_SOURCES and not (only and source in only)):
            continue
        name = CORPUS_NAME.get(source, source)
        out_dir = shard_dir / (name + suffix)
        tag = "_w%02d" % worker_id if fan_out else ""
        manifest = out_dir / ("manifest.w%02d.yaml" % worker_id if fan_out else "manifest.yaml")
        if manifest.is_file():
            log("[%s] %s exists, skipping" % (source, manifest.name))
            done[source] = str(manifest)
            continue
        raw = raw_dir / (name + tag + ".jsonl")
        if pull_fn is not None:
            have, _ = pull_fn(raw, n, source)
        else:
            share = -(-n // num_workers) if fan_out else n
            streams = source_streams(source, share, workers=concurrency.get(source, 64), worker_id=worker_id, num_workers=num_workers)
            have, _ = pull(raw, share, streams, log=log)
        log("[%s] %d documents in %s" % (source, have, raw))
        mark = _note(raw, "shuffled")
        if not mark.is_file():
            tmp = Path(str(raw) + ".shuffling")
            lines = shuffle_jsonl(raw, tmp, seed=shuffle_seed)
            os.replace(tmp, raw)
            mark.write_text(json.dumps({"seed": shuffle_seed, "buckets": 64, "lines": lines}))
        shard_source(raw, tokenizer, out_dir, name, workers=workers, prefix_tag=tag, manifest_name=manifest.name)
        done[source] = str(manifest)
        if delete_raw:
            for p in (raw, mark, _note(raw, "scanned"), _note(raw, "revision")):
                if p.exists():
                    p.unlink()
    return done


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("shuffle"); s.add_argument("src"); s.add_argument("dst"); s.add_argument("--seed", type=int, default=0)
    s.add_argument("--buckets", type=int, default=64)
    p = sub.add_parser("plan"); p.add_argument("src"); p.add_argument("--workers", type=int, default=8)
    h = sub.add_parser("shard"); h.add_argument("src"); h.add_argument("--tokenizer", required=True); h.add_argument("--out-dir", required=True)
    h.add_argument("--name", required=True); h.add_argument("--workers", type=int, default=8); h.add_argument("--shard-bytes", type=int, default=1 << 30)
    h.add_argument("--field", default="text")
    q = sub.add_parser("pull"); q.add_argument("source", choices=sorted(PULL_SOURCES)); q.add_argument("--docs", type=int, required=True)
    q.add_argument("--raw-dir", default="data/raw"); q.add_argument("--concurrency", type=int, default=64)
    b = sub.add_parser("build"); b.add_argument("--preset", choices=sorted(PRESETS))
    for src in PULL_SOURCES:
        b.add_argument("--docs-" + src.split("_")[0], type=int, dest="docs_" + src)
    b.add_argument("--tokenizer", default="data/tokenizer.json"); b.add_argument("--raw-dir", default="data/raw"); b.add_argument("--shard-dir", default="data/shards")
    b.add_argument("--shard-suffix", default="_proxy"); b.add_argument("--delete-raw", action="store_true"); b.add_argument("--shuffle-seed", type=int, default=0)
    b.add_argument("--only", nargs="+", choices=sorted(set(PULL_SOURCES) | set(CORPUS_NAME.values())),
                   help="restrict to these sources (default: the four pretraining sources; dolma3_dolmino_mix runs only when named here)")
    b.add_argument("--workers", type=int, default=8, help="tokenizer processes of the shard step")
    b.add_argument("--stack-concurrency", type=int, default=64, help="parallel blob fetches for the Stack")
    b.add_argument("--dolma3-concurrency", type=int, default=24, help="parallel file fetches for dolma3_dolmino_mix")
    b.add_argument("--dolma3-shard-workers", type=int, default=8, help="tokenizer processes for dolma3_dolmino_mix's shard step")
    b.add_argument("--worker-id", type=int, default=0, help="zero-based index of this machine in a Stack fan-out")
    b.add_argument("--num-workers", type=int, default=1, help="machines of the Stack fan-out (1: no slicing); needs --only stack_v2_permissive")
    argv = sys.argv[1:]
    if argv and argv[0].startswith("--") and argv[0] != "--help":   # `build_corpus.py --preset ...`: the orchestration is the default command
        argv = ["build"] + argv
    a = ap.parse_args(argv)
    if a.cmd == "shuffle":
        print(json.dumps({"lines": shuffle_jsonl(a.src, a.dst, a.seed, a.buckets)}))
    elif a.cmd == "plan":
        print(json.dumps(segment_plan(a.src, a.workers), indent=1))
    elif a.cmd == "shard":
        m = shard_source(a.src, a.tokenizer, a.out_dir, a.name, a.workers, a.shard_bytes, a.field)
        print(json.dumps({"shards": len(m.shards), "documents": m.total_documents, "tokens": m.total_tokens}))
    elif a.cmd == "pull":
        try:
            have, scanned = pull(Path(a.raw_dir) / (a.source + ".jsonl"), a.docs, source_streams(a.source, a.docs, workers=a.concurrency),
                                 log=lambda m: print(m, file=sys.stderr))
        except ImportError as e:
            print("pull %s: %s is not installed (the pullers need `datasets`, `huggingface_hub`, and `boto3` for the Stack)" % (a.source, e.name), file=sys.stderr)
            return 2
        print(json.dumps({"documents": have, "scanned": scanned}))
    else:
        counts = dict(PRESETS.get(a.preset) or {})
        for src in PULL_SOURCES:
            if getattr(a, "docs_" + src) is not None:
                counts[src] = getattr(a, "docs_" + src)
        if not counts:
            ap.error("build needs --preset or at least one --docs-<source>")
        try:
            if a.num_workers > 1 and not 0 <= a.worker_id < a.num_workers:
                ap.error("--worker-id=%d out of range for --num-workers=%d" % (a.worker_id, a.num_workers))
            only = [SHORT_NAME.get(x, x) for x in a.only] if a.only else None
            workers = a.dolma3_shard_workers if only == ["dolma3_dolmino_mix"] else a.workers
            print(json.dumps(build(counts, a.raw_dir, a.shard_dir, a.tokenizer, a.shard_suffix, a.shuffle_seed, workers, a.delete_raw, only,
                                   log=lambda m: print(m, file=sys.stderr), concurrency={"stack": a.stack_concurrency, "dolma3_dolmino_mix": a.dolma3_concurrency},
                                   worker_id=a.worker_id, num_workers=a.num_workers)))
        except ValueError as e:
            ap.error(str(e))
        except ImportError as e:
            print("build: %s is not installed (the pullers need `datasets`, `huggingface_hub`, and `boto3` for the Stack)" % e.name, file=sys.stderr)
            return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
