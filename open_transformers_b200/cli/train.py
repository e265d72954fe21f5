"""``pretrain-train --config-name NAME [--resume-from DIR] [key=value overrides]``
(reference src/pretrain/cli/train.py:25-50)."""
from __future__ import annotations

import argparse
import json
import logging
import sys


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-train")
    ap.add_argument("--config-name", required=True)
    ap.add_argument("--resume-from")
    ap.add_argument("--device", default=None, choices=[None, "cuda", "cpu"])
    ap.add_argument("--data-root")
    ap.add_argument("--max-steps", type=int)
    ap.add_argument("--synthetic-data", action="store_true", help="create missing sources as seed-generated uniform-random shards")
    ap.add_argument("overrides", nargs="*")
    from ._args import parse_with_overrides

    a = parse_with_overrides(ap, argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(message)s")
    from ..config import load_config
    from ..train.loop import train

    cfg = load_config(a.config_name, a.overrides)
    if a.synthetic_data:
        import os

        from ..data.synthetic import ensure_synthetic_sources

        if int(os.environ.get("RANK", "0")) == 0:
            ensure_synthetic_sources(cfg, a.data_root or ".", cfg.train.total_tokens)
    from ..parallel.env import shutdown_distributed

    res = train(cfg, a.resume_from, device=a.device, data_root=a.data_root, max_steps=a.max_steps)
    shutdown_distributed()  # after a clean run only: a barrier, then the process group is destroyed (a failed rank's peers may be gone)
    import os

    if int(os.environ.get("RANK", "0")) == 0:  # one line per run: lines of several ranks would run together on a shared pipe
        print(json.dumps({k: v for k, v in res.items() if k != "losses"}, default=str), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
