"""``pretrain-fetch-audit-data --checkpoint DIR --mirror gs://... | DIR --dest DIR [--until-step N]``:
download (and verify) only the shards an audit interval reads; see data/fetch_interval.py."""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-fetch-audit-data")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--mirror", "--gcs-root", dest="mirror", required=True)
    ap.add_argument("--dest", required=True)
    ap.add_argument("--until-step", type=int)
    a = ap.parse_args(argv)
    from ..data.fetch_interval import fetch_audit_interval

    print(fetch_audit_interval(a.checkpoint, a.mirror, a.dest, until_step=a.until_step))
    return 0


if __name__ == "__main__":
    sys.exit(main())
