"""``pretrain-prepare-data <subcommand>``: train-tokenizer | shard | merge-manifests | inspect | token-stats |
synthetic | replay-step (reference src/pretrain/cli/prepare_data.py:300-378)."""
from __future__ import annotations

import argparse
import json
import sys


def _inputs(a) -> list[str]:
    """Input files of a subcommand: the positional paths, or ``--input-dir`` / ``--glob`` (the reference's form)."""
    from pathlib import Path

    paths = list(a.inputs or [])
    if a.input_dir:
        pattern = a.glob or ("*.jsonl" if a.format == "jsonl" else "*.parquet")
        found = sorted(str(p) for p in Path(a.input_dir).glob(pattern))
        if not found:
            raise SystemExit("no input files matched %s/%s" % (a.input_dir, pattern))
        paths += found
    if not paths:
        raise SystemExit("give input files or --input-dir")
    return paths


def cmd_train_tokenizer(a) -> int:
    from ..data.prepare import iter_texts
    from ..data.tokenizer import compute_hash, train_tokenizer

    out = train_tokenizer(iter_texts(_inputs(a), a.field), a.output, a.vocab_size, a.min_frequency)
    print(json.dumps({"tokenizer": str(out), "hash": compute_hash(out)}))
    return 0


def cmd_shard(a) -> int:
    from ..data.prepare import iter_jsonl_segment, iter_jsonl_worker_share, iter_texts, write_shards
    from ..data.tokenizer import Tokenizer

    if not a.out_dir or not a.name:
        raise SystemExit("shard needs --output-dir and --source-name")
    if a.num_workers > 1 and a.shard_tag:
        raise SystemExit("pass --num-workers (input segmenting and automatic tagging) OR --shard-tag (output naming only), not both")
    inputs = _inputs(a)
    tok = Tokenizer(a.tokenizer)
    tag, manifest_name = "", "manifest.yaml"
    if a.segment:
        start, end = (int(x) for x in a.segment.split(":"))
        texts = iter_jsonl_segment(inputs[0], start, end, a.field)
    elif a.num_workers > 1:
        if any(not str(p).endswith((".jsonl", ".json")) for p in inputs):
            raise SystemExit("--num-workers > 1 splits jsonl inputs by byte range; parquet inputs are already one file per worker")
        if not 0 <= a.worker_id < a.num_workers:
            raise SystemExit("--worker-id=%d out of range for --num-workers=%d" % (a.worker_id, a.num_workers))
        texts = iter_jsonl_worker_share(inputs, a.worker_id, a.num_workers, a.field)
        tag, manifest_name = "_w%02d" % a.worker_id, "manifest.w%02d.yaml" % a.worker_id
    else:
        texts = iter_texts(inputs, a.field)
        if a.shard_tag:
            tag, manifest_name = "_" + a.shard_tag, "manifest.%s.yaml" % a.shard_tag
    raw = [p for p in inputs if str(p).endswith((".jsonl", ".json"))]   # digests of the raw jsonl inputs go into the manifest
    man = write_shards(texts, tok, a.out_dir, a.name, shard_bytes=a.shard_bytes, raw_inputs=raw, prefix_tag=tag, manifest_name=manifest_name)
    print(json.dumps({"shards": len(man.shards), "documents": man.total_documents, "tokens": man.total_tokens, "manifest": manifest_name}))
    return 0


def cmd_merge(a) -> int:
    from ..data.manifest import SourceManifest
    from ..data.prepare import merge_manifests, merge_worker_manifests

    if a.output_dir:   # the fan-out form: manifest.w*.yaml of one directory -> its manifest.yaml
        try:
            merged = merge_worker_manifests(a.output_dir, a.expected_workers, a.remove_worker_manifests)
        except ValueError as e:
            raise SystemExit(str(e))
    else:
        if not (a.manifests and a.name and a.output):
            raise SystemExit("merge-manifests needs --output-dir, or manifest files with --name and --output")
        merged = merge_manifests([SourceManifest.load(p) for p in a.manifests], a.name)
        merged.save(a.output)
    print(json.dumps({"shards": len(merged.shards), "documents": merged.total_documents, "tokens": merged.total_tokens}))
    return 0


def cmd_inspect(a) -> int:
    from ..data.prepare import inspect_shard
    from ..data.tokenizer import Tokenizer

    prefix = a.shard or a.prefix
    if not prefix:
        raise SystemExit("inspect needs a shard prefix (positional or --shard)")
    print(json.dumps(inspect_shard(prefix, Tokenizer(a.tokenizer) if a.tokenizer else None, a.docs), indent=1, default=str))
    return 0


def cmd_token_stats(a) -> int:
    from ..data.manifest import SourceManifest

    if a.sample:       # bytes per token of a text sample under a tokenizer
        from pathlib import Path

        from ..data.prepare import bytes_per_token
        from ..data.tokenizer import Tokenizer

        if not a.tokenizer:
            raise SystemExit("token-stats --sample needs --tokenizer")
        print(json.dumps({"bytes_per_token": bytes_per_token(Tokenizer(a.tokenizer), Path(a.sample).read_text(encoding="utf-8"))}, indent=2))
        return 0
    rows = []
    for p in a.manifests:
        m = SourceManifest.load(p)
        rows.append({"name": m.name, "shards": len(m.shards), "documents": m.total_documents, "tokens": m.total_tokens,
                     "mean_doc_len": m.total_tokens / max(m.total_documents, 1)})
    total = sum(r["tokens"] for r in rows)
    for r in rows:
        r["token_share"] = r["tokens"] / max(total, 1)
    print(json.dumps(rows, indent=1))
    return 0


def cmd_synthetic(a) -> int:
    if not a.config_name:   # the reference's form: two sources of random documents, no configuration involved
        from ..data.prepare import write_random_sources

        made = write_random_sources(a.output_dir, a.docs_a, a.docs_b, a.min_doc_len, a.max_doc_len, a.vocab_size, a.seed)
        print(json.dumps({"output_dir": a.output_dir, "sources": {m.name: {"documents": m.total_documents, "tokens": m.total_tokens} for m in made}}))
        return 0
    from ..config import load_config
    from ..data.synthetic import ensure_synthetic_sources

    cfg = load_config(a.config_name, a.overrides)
    ensure_synthetic_sources(cfg, a.data_root, a.tokens or cfg.train.total_tokens)
    print(json.dumps({"data_root": a.data_root, "sources": [s.path for s in cfg.data.sources]}))
    return 0


def cmd_replay_step(a) -> int:
    """Print the windows (token ids, and text when a tokenizer is given) that a given step trains on."""
    from ..config import load_config
    from ..data.loader import build_global_loader

    cfg = load_config(a.config_name, list(a.overrides) + list(a.override or []))
    V = a.world_size or cfg.run.virtual_dp_size or max(cfg.run.dp_shard_size, 1) * cfg.run.dp_replicate_size
    ranks = [a.rank] if a.rank is not None else list(range(V))
    view = build_global_loader(cfg, ranks, V, data_root=a.data_root, seed=a.seed)
    tok = None
    if a.tokenizer:
        from ..data.tokenizer import Tokenizer

        tok = Tokenizer(a.tokenizer)
    for plan, batches in view:
        if plan.step == a.step:
            for r, k, w in batches:
                for slot in range(w.shape[0]):
                    print(json.dumps({"step": plan.step, "dp_rank": r, "accum": k, "slot": slot, "tokens": w[slot][:a.max_tokens].tolist(),
                                      "text": tok.decode(w[slot][:a.max_tokens]) if tok else None}))
            return 0
    return 1


def main(argv=None) -> int:
    """Every subcommand takes the reference's flags (src/pretrain/cli/prepare_data.py:300-378) and, beside them, the shorter
    positional forms this package's scripts use."""
    ap = argparse.ArgumentParser(prog="pretrain-prepare-data")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def io_flags(p):
        p.add_argument("inputs", nargs="*", help="input files (or use --input-dir)")
        p.add_argument("--input-dir")
        p.add_argument("--glob", default=None, help="with --input-dir (default: *.parquet, *.jsonl with --format jsonl)")
        p.add_argument("--format", choices=["parquet", "jsonl"], default="parquet")
        p.add_argument("--text-field", "--field", dest="field", default="text")

    p = sub.add_parser("train-tokenizer", help="train a fresh byte-level BPE tokenizer")
    io_flags(p)
    p.add_argument("--output", required=True)
    p.add_argument("--vocab-size", type=int, default=128_256)
    p.add_argument("--min-frequency", type=int, default=2)
    p.set_defaults(fn=cmd_train_tokenizer)

    p = sub.add_parser("shard", help="parquet / jsonl -> indexed binary shards with a manifest")
    io_flags(p)
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--output-dir", "--out-dir", dest="out_dir")
    p.add_argument("--source-name", "--name", dest="name")
    p.add_argument("--shard-bytes", type=int, default=1 << 30)
    p.add_argument("--worker-id", type=int, default=0, help="zero-based worker index of a fan-out")
    p.add_argument("--num-workers", type=int, default=1, help="fan-out size: each worker reads its byte range of the jsonl inputs and writes "
                                                               "<source>_w<K>_* shards and manifest.w<K>.yaml (join with merge-manifests)")
    p.add_argument("--shard-tag", default="", help="output naming only (e.g. w03): <source>_<tag>_* and manifest.<tag>.yaml, for workers "
                                                   "that each have their own input")
    p.add_argument("--segment", help="start:end byte range of a single jsonl input")
    p.set_defaults(fn=cmd_shard)

    p = sub.add_parser("merge-manifests", help="join per-worker manifest.w*.yaml into manifest.yaml")
    p.add_argument("manifests", nargs="*")
    p.add_argument("--name")
    p.add_argument("--output")
    p.add_argument("--output-dir", help="directory holding the workers' manifest.w*.yaml")
    p.add_argument("--expected-workers", type=int, default=0, help="fail unless exactly this many worker manifests are found")
    p.add_argument("--remove-worker-manifests", action="store_true")
    p.set_defaults(fn=cmd_merge)

    p = sub.add_parser("inspect", help="decode a few documents of a shard")
    p.add_argument("prefix", nargs="?")
    p.add_argument("--shard", help="shard prefix (no .bin / .idx)")
    p.add_argument("--tokenizer")
    p.add_argument("--n", "--docs", dest="docs", type=int, default=3)
    p.set_defaults(fn=cmd_inspect)

    p = sub.add_parser("token-stats", help="bytes per token of a sample, or token shares of manifests")
    p.add_argument("manifests", nargs="*")
    p.add_argument("--tokenizer")
    p.add_argument("--sample", help="path of a UTF-8 text file")
    p.set_defaults(fn=cmd_token_stats)

    p = sub.add_parser("synthetic", help="seed-generated sources: of a configuration (--config-name), or two sources of random documents")
    p.add_argument("--config-name")
    p.add_argument("--data-root", default=".")
    p.add_argument("--tokens", type=int)
    p.add_argument("--output-dir", default="data/shards/synthetic")
    p.add_argument("--docs-a", type=int, default=2000)
    p.add_argument("--docs-b", type=int, default=1000)
    p.add_argument("--min-doc-len", type=int, default=64)
    p.add_argument("--max-doc-len", type=int, default=512)
    p.add_argument("--vocab-size", type=int, default=128_256)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("overrides", nargs="*")
    p.set_defaults(fn=cmd_synthetic)

    p = sub.add_parser("replay-step", help="print the windows step N trains on")
    p.add_argument("--config-name", required=True)
    p.add_argument("--data-root", default=".")
    p.add_argument("--step", type=int, required=True)
    p.add_argument("--seed", type=int, default=None, help="stream seed (default: the configuration's run.seed)")
    p.add_argument("--rank", type=int, default=None, help="only this data-parallel rank's windows")
    p.add_argument("--world-size", type=int, default=None, help="data-parallel size the ranks refer to (default: the configured one)")
    p.add_argument("--override", nargs="*", default=[])
    p.add_argument("--tokenizer")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("overrides", nargs="*")
    p.set_defaults(fn=cmd_replay_step)
    from ._args import parse_with_overrides

    cmd = next((x for x in (argv if argv is not None else sys.argv[1:]) if not str(x).startswith("-")), None)
    a = parse_with_overrides(ap, argv) if cmd in ("synthetic", "replay-step") else ap.parse_args(argv)  # only two subcommands take overrides
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
