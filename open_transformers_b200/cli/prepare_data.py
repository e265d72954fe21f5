"""``pretrain-prepare-data <subcommand>``: train-tokenizer | shard | merge-manifests | inspect | token-stats |
synthetic | replay-step (reference src/pretrain/cli/prepare_data.py:300-378)."""
from __future__ import annotations

import argparse
import json
import sys


def cmd_train_tokenizer(a) -> int:
    from ..data.prepare import iter_texts
    from ..data.tokenizer import compute_hash, train_tokenizer

    out = train_tokenizer(iter_texts(a.inputs, a.field), a.output, a.vocab_size, a.min_frequency)
    print(json.dumps({"tokenizer": str(out), "hash": compute_hash(out)}))
    return 0


def cmd_shard(a) -> int:
    from ..data.prepare import iter_jsonl_segment, iter_texts, write_shards
    from ..data.tokenizer import Tokenizer

    tok = Tokenizer(a.tokenizer)
    if a.segment:
        start, end = (int(x) for x in a.segment.split(":"))
        texts = iter_jsonl_segment(a.inputs[0], start, end, a.field)
    else:
        texts = iter_texts(a.inputs, a.field)
    man = write_shards(texts, tok, a.out_dir, a.name, shard_bytes=a.shard_bytes, raw_inputs=a.inputs)
    print(json.dumps({"shards": len(man.shards), "documents": man.total_documents, "tokens": man.total_tokens}))
    return 0


def cmd_merge(a) -> int:
    from ..data.manifest import SourceManifest
    from ..data.prepare import merge_manifests

    merged = merge_manifests([SourceManifest.load(p) for p in a.manifests], a.name)
    merged.save(a.output)
    print(json.dumps({"shards": len(merged.shards), "tokens": merged.total_tokens}))
    return 0


def cmd_inspect(a) -> int:
    from ..data.prepare import inspect_shard
    from ..data.tokenizer import Tokenizer

    print(json.dumps(inspect_shard(a.prefix, Tokenizer(a.tokenizer) if a.tokenizer else None, a.docs), indent=1, default=str))
    return 0


def cmd_token_stats(a) -> int:
    from ..data.manifest import SourceManifest

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

    cfg = load_config(a.config_name, a.overrides)
    V = cfg.run.virtual_dp_size or max(cfg.run.dp_shard_size, 1) * cfg.run.dp_replicate_size
    view = build_global_loader(cfg, list(range(V)), V, data_root=a.data_root)
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
    ap = argparse.ArgumentParser(prog="pretrain-prepare-data")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("train-tokenizer"); p.add_argument("inputs", nargs="+"); p.add_argument("--output", required=True)
    p.add_argument("--vocab-size", type=int, default=128_256); p.add_argument("--min-frequency", type=int, default=2); p.add_argument("--field", default="text")
    p.set_defaults(fn=cmd_train_tokenizer)
    p = sub.add_parser("shard"); p.add_argument("inputs", nargs="+"); p.add_argument("--tokenizer", required=True); p.add_argument("--out-dir", required=True)
    p.add_argument("--name", required=True); p.add_argument("--shard-bytes", type=int, default=1 << 30); p.add_argument("--field", default="text")
    p.add_argument("--segment", help="start:end byte range of a single jsonl input (fan-out workers)"); p.set_defaults(fn=cmd_shard)
    p = sub.add_parser("merge-manifests"); p.add_argument("manifests", nargs="+"); p.add_argument("--name", required=True); p.add_argument("--output", required=True)
    p.set_defaults(fn=cmd_merge)
    p = sub.add_parser("inspect"); p.add_argument("prefix"); p.add_argument("--tokenizer"); p.add_argument("--docs", type=int, default=3); p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("token-stats"); p.add_argument("manifests", nargs="+"); p.set_defaults(fn=cmd_token_stats)
    p = sub.add_parser("synthetic"); p.add_argument("--config-name", required=True); p.add_argument("--data-root", default="."); p.add_argument("--tokens", type=int)
    p.add_argument("overrides", nargs="*"); p.set_defaults(fn=cmd_synthetic)
    p = sub.add_parser("replay-step"); p.add_argument("--config-name", required=True); p.add_argument("--data-root", default="."); p.add_argument("--step", type=int, required=True)
    p.add_argument("--tokenizer"); p.add_argument("--max-tokens", type=int, default=64); p.add_argument("overrides", nargs="*"); p.set_defaults(fn=cmd_replay_step)
    from ._args import parse_with_overrides

    a = ap.parse_known_args(argv)[0]
    a = parse_with_overrides(ap, argv) if hasattr(a, "overrides") else ap.parse_args(argv)  # only two subcommands take overrides
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
