"""``pretrain-inspect-checkpoint DIR``: print meta.json and the side files of a checkpoint."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-inspect-checkpoint")
    ap.add_argument("checkpoint")
    ap.add_argument("--full-config", action="store_true")
    a = ap.parse_args(argv)
    d = Path(a.checkpoint)
    meta = json.loads((d / "meta.json").read_text())
    if not a.full_config and meta.get("config_resolved"):
        meta["config_resolved"] = "<%d bytes, --full-config to print>" % len(meta["config_resolved"])
    print(json.dumps(meta, indent=1, sort_keys=True))
    print("complete:", (d / "_COMPLETE").exists())
    if (d / "state_hash.txt").exists():
        print("state_hash:", (d / "state_hash.txt").read_text().strip())
    print("files:", ", ".join(sorted(p.name for p in d.iterdir())))
    return 0


if __name__ == "__main__":
    sys.exit(main())
