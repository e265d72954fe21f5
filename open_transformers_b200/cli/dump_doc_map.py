"""``pretrain-dump-doc-map``: which documents fed which optimizer step (a data explorer for a finished or running run).

    pretrain-dump-doc-map --checkpoint runs/<id>/checkpoints/step_000080957 --out-dir DIR [--data-root data/shards]
                          [--until-step N] [--chunk-steps 1000] [--from-checkpoint-state] [--config-name NAME]
                          [--dp-world-size V]

The canonical stream is walked over document LENGTHS (manifests and ``.idx`` files; no token payload, no model), and every
piece of a document that lands in a training window becomes one Parquet row: step, window, micro-batch, slot, virtual rank,
source, shard, document, token range (``data/doc_map.py``).

Two ways to walk. The default starts at the first step of the run and stops before the checkpoint's step; the position the
walk ends at must then equal the checkpoint's ``global_stream.json``, and the command exits 2 if it does not (the map would
describe another run). ``--from-checkpoint-state`` starts where the checkpoint stands and needs ``--until-step`` beyond it;
a checkpoint whose next window begins with tokens left over from the previous step cannot be a starting point, because
those tokens no longer say which document they came from.
(flag set: reference src/pretrain/cli/dump_doc_map.py:31-55)
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
    ap = argparse.ArgumentParser(prog="pretrain-dump-doc-map", description="Write the step -> document map of a run as Parquet files.")
    ap.add_argument("--checkpoint", required=True, help="a checkpoint of the run: its meta.json names seed, topology and step")
    ap.add_argument("--out-dir", required=True, help="where step_docs-<first>-<last>.parquet and step_docs_manifest.json go")
    ap.add_argument("--data-root", default=None, help="parent of the sources' directories, if they are not where the configuration says")
    ap.add_argument("--config-name", default=None, help="named configuration to use in place of the one stored in the checkpoint")
    ap.add_argument("--until-step", type=int, default=None, help="first step NOT to map; default: the checkpoint's own step")
    ap.add_argument("--chunk-steps", type=int, default=1000, help="how many steps share one Parquet file")
    ap.add_argument("--from-checkpoint-state", action="store_true",
                    help="begin at the checkpoint's stream position rather than at step 0; --until-step must then be given")
    ap.add_argument("--dp-world-size", type=int, default=None, help="number of virtual ranks, if not the checkpoint's")
    return ap


def resolve_until_step(until_step: int | None, checkpoint_step: int, *, from_checkpoint_state: bool) -> int:
    """First step the walk leaves out. Walking from the start, no flag means "up to the checkpoint", the one end point whose
    position can be checked. Walking from the checkpoint, that default would be an empty walk that still exits 0 - so the
    caller has to name an end, and one that lies ahead."""
    if from_checkpoint_state and until_step is None:
        raise SystemExit("--from-checkpoint-state: say where to stop with --until-step (the start is step %d)" % checkpoint_step)
    if from_checkpoint_state and until_step <= checkpoint_step:
        raise SystemExit("--until-step %d does not lie after the checkpoint's step %d: the walk would be empty" % (until_step, checkpoint_step))
    return checkpoint_step if until_step is None else until_step


def open_walk(cfg, desc: dict, *, data_root, seed: int, resume: bool):
    """The index-only window view the map is read from: a fresh stream, or one restored to the checkpoint's position."""
    from ..data.global_stream import GlobalStreamState
    from ..data.loader import build_global_loader
    from ..data.mix_sampler import clear_caches

    clear_caches()
    if not resume:
        return build_global_loader(cfg, [], 1, data_root=data_root, index_only=True, seed=seed)
    meta = desc["meta"]
    if desc["stream"] is None:
        raise SystemExit("--from-checkpoint-state: the checkpoint stores no global_stream.json")
    view = build_global_loader(cfg, [], 1, state=GlobalStreamState.from_json(desc["stream"]), consumed_tokens=int(meta["consumed_tokens"]),
                               start_step=int(meta["step"]), data_root=data_root, index_only=True, seed=seed)
    if view.has_carry_over:
        raise SystemExit("the checkpoint's next window starts with left-over tokens of the step before, whose documents are no longer "
                         "known; map this run from step 0 instead (omit --from-checkpoint-state)")
    return view


def run(a) -> int:
    from ..data.doc_map import compare_position, write_doc_map, write_manifest
    from ..data.fetch_interval import load_run_config, read_checkpoint_descriptor

    ckpt = Path(a.checkpoint)
    desc = read_checkpoint_descriptor(ckpt)
    meta = desc["meta"]
    here = int(meta["step"])
    cfg = load_run_config(meta, a.config_name)
    stop = resolve_until_step(a.until_step, here, from_checkpoint_state=a.from_checkpoint_state)
    seed, ranks = int(meta.get("seed", cfg.run.seed)), int(a.dp_world_size or meta["dp_world_size"])
    view = open_walk(cfg, desc, data_root=a.data_root, seed=seed, resume=a.from_checkpoint_state)
    names = [w.name for w in view._core.walkers]
    log.info("mapping steps %s..%d of seed %d for %d virtual ranks, micro-batch %d, sources %s", here if a.from_checkpoint_state else 0,
             stop - 1, seed, ranks, cfg.train.micro_batch_size, names)
    began = time.time()
    summary = write_doc_map(view, a.out_dir, until_step=stop, micro_batch_size=cfg.train.micro_batch_size, dp_world_size=ranks,
                            chunk_steps=a.chunk_steps,
                            progress=lambda step, rows: log.info("step %d / %d, %d rows, %.0fs", step, stop, rows, time.time() - began))
    record = {"checkpoint": str(ckpt), "git_sha": meta.get("git_sha"), "seed": seed, "dp_world_size": ranks,
              "micro_batch_size": cfg.train.micro_batch_size, "seq_len": cfg.train.seq_len, "sources": names,
              "elapsed_s": round(time.time() - began, 1)}
    status = 0
    checkable = stop == here and not a.from_checkpoint_state and desc["stream"] is not None
    if checkable:
        differences = compare_position(summary["position"], desc["stream"])
        record["validation"] = {"against": str(ckpt / "global_stream.json"), "match": not differences, "problems": differences}
        if differences:
            status = 2
            log.error("the walk does not end where %s says the run stood: %s", ckpt.name, differences)
        else:
            log.info("the walk ends exactly at the position recorded in %s", ckpt.name)
    where = write_manifest(a.out_dir, summary, record)
    shown = dict(summary, **record)
    shown.pop("files", None)
    print(json.dumps(shown, indent=2))
    print("manifest: %s" % where)
    return status


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
