"""``pretrain-dump-doc-map``: the step -> document map of a run (training data explorer).

    pretrain-dump-doc-map --checkpoint runs/<id>/checkpoints/step_000080957 --out-dir DIR [--data-root data/shards]
                          [--until-step N] [--chunk-steps 1000] [--from-checkpoint-state] [--config-name NAME]
                          [--dp-world-size V]

Replays the canonical stream by document lengths only - from step 0, or with ``--from-checkpoint-state`` from the
checkpoint's stream position - and writes one Parquet row per document piece per window (``data/doc_map.py``). Reads
``manifest.yaml`` and ``.idx`` files only. From step 0 the walk ends at the checkpoint's step by default, and when it does
its final stream position is compared with the checkpoint's ``global_stream.json``: a difference exits 2.
(flags and behaviour: reference src/pretrain/cli/dump_doc_map.py:31-157)
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import time
from pathlib import Path

log = logging.getLogger("pretrain.dump_doc_map")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pretrain-dump-doc-map")
    ap.add_argument("--checkpoint", required=True, help="checkpoint directory (meta.json and, for the position check, global_stream.json)")
    ap.add_argument("--out-dir", required=True, help="directory for step_docs-*.parquet and step_docs_manifest.json")
    ap.add_argument("--data-root", default=None, help="directory holding one <source>/ per source (default: the configured paths, relative to the cwd)")
    ap.add_argument("--config-name", default=None, help="train config name (default: the configuration recorded in meta.json)")
    ap.add_argument("--until-step", type=int, default=None, help="walk steps < N (default: the checkpoint's step)")
    ap.add_argument("--chunk-steps", type=int, default=1000, help="steps per Parquet file")
    ap.add_argument("--from-checkpoint-state", action="store_true",
                    help="start at the checkpoint's stream position instead of step 0 (then --until-step is required); refused when the "
                         "checkpoint carries tokens over into its next window, because those name no document")
    ap.add_argument("--dp-world-size", type=int, default=None, help="override meta.json's dp_world_size")
    return ap


def resolve_until_step(until_step: int | None, checkpoint_step: int, *, from_checkpoint_state: bool) -> int:
    """Exclusive end of the walk. From step 0 the default is the checkpoint's step (which arms the position check). From the
    checkpoint's state that default would walk nothing, so the flag must name a step past the start."""
    if not from_checkpoint_state:
        return checkpoint_step if until_step is None else until_step
    if until_step is None:
        raise SystemExit("--from-checkpoint-state needs --until-step (the walk starts at the checkpoint's step)")
    if until_step <= checkpoint_step:
        raise SystemExit("--until-step %d is not past the checkpoint's step %d; nothing to walk" % (until_step, checkpoint_step))
    return until_step


def run(a) -> int:
    from ..config import load_config, parse_config_resolved
    from ..data.doc_map import compare_position, write_doc_map, write_manifest
    from ..data.fetch_interval import read_checkpoint_descriptor
    from ..data.global_stream import GlobalStreamState
    from ..data.loader import build_global_loader
    from ..data.mix_sampler import clear_caches

    ckpt = Path(a.checkpoint)
    desc = read_checkpoint_descriptor(ckpt)
    meta = desc["meta"]
    cfg = load_config(a.config_name) if a.config_name else parse_config_resolved(meta["config_resolved"])
    seed = int(meta.get("seed", cfg.run.seed))
    dp_world = int(a.dp_world_size or meta["dp_world_size"])
    until = resolve_until_step(a.until_step, int(meta["step"]), from_checkpoint_state=a.from_checkpoint_state)
    mb = cfg.train.micro_batch_size
    clear_caches()
    if a.from_checkpoint_state:
        if desc["stream"] is None:
            raise SystemExit("checkpoint %s has no global_stream.json to start from" % ckpt)
        view = build_global_loader(cfg, [], 1, state=GlobalStreamState.from_json(desc["stream"]), consumed_tokens=int(meta["consumed_tokens"]),
                                   start_step=int(meta["step"]), data_root=a.data_root, index_only=True, seed=seed)
        if view.has_carry_over:
            raise SystemExit("checkpoint %s carries tokens over from the previous step; they name no document. "
                             "Drop --from-checkpoint-state and walk from step 0." % ckpt)
    else:
        view = build_global_loader(cfg, [], 1, data_root=a.data_root, index_only=True, seed=seed)
    sources = [w.name for w in view._core.walkers]
    log.info("seed=%d dp_world=%d micro_batch=%d until_step=%d sources=%s", seed, dp_world, mb, until, sources)
    t0 = time.time()
    summary = write_doc_map(view, a.out_dir, until_step=until, micro_batch_size=mb, dp_world_size=dp_world, chunk_steps=a.chunk_steps,
                            progress=lambda step, rows: log.info("step %d / %d, %d rows, %.0fs", step, until, rows, time.time() - t0))
    extra = {"checkpoint": str(ckpt), "git_sha": meta.get("git_sha"), "seed": seed, "dp_world_size": dp_world, "micro_batch_size": mb,
             "seq_len": cfg.train.seq_len, "sources": sources, "elapsed_s": round(time.time() - t0, 1)}
    rc = 0
    if until == int(meta["step"]) and not a.from_checkpoint_state and desc["stream"] is not None:
        problems = compare_position(summary["position"], desc["stream"])
        extra["validation"] = {"against": str(ckpt / "global_stream.json"), "match": not problems, "problems": problems}
        if problems:
            log.error("stream position does NOT match the checkpoint: %s", problems)
            rc = 2
        else:
            log.info("stream position matches checkpoint %s", ckpt.name)
    path = write_manifest(a.out_dir, summary, extra)
    print(json.dumps({k: v for k, v in {**summary, **extra}.items() if k != "files"}, indent=2))
    print("manifest: %s" % path)
    return rc


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
