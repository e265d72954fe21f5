"""``pretrain-dump-doc-map``: write the step -> document Parquet map for a range of steps of a config
(from step 0) or of a checkpoint's stream position."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-dump-doc-map")
    ap.add_argument("--config-name")
    ap.add_argument("--checkpoint")
    ap.add_argument("--data-root", default=".")
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("overrides", nargs="*")
    from ._args import parse_with_overrides

    a = parse_with_overrides(ap, argv)
    from ..config import load_config, parse_config_resolved
    from ..data.doc_map import write_doc_map
    from ..data.global_stream import GlobalStreamState
    from ..data.loader import build_global_loader

    state, consumed, step = None, 0, 0
    if a.checkpoint:
        meta = json.loads((Path(a.checkpoint) / "meta.json").read_text())
        cfg = parse_config_resolved(meta["config_resolved"])
        state = GlobalStreamState.from_json(json.loads((Path(a.checkpoint) / "global_stream.json").read_text()))
        consumed, step, V = meta["consumed_tokens"], meta["step"], meta["dp_world_size"]
    else:
        cfg = load_config(a.config_name, a.overrides)
        V = cfg.run.virtual_dp_size or max(cfg.run.dp_shard_size, 1) * cfg.run.dp_replicate_size
    view = build_global_loader(cfg, [], V, state=state, consumed_tokens=consumed, start_step=step, data_root=a.data_root)
    n = write_doc_map(view, a.steps, V, a.output)
    print(json.dumps({"rows": n, "output": a.output}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
