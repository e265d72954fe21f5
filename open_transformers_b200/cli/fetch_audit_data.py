"""``pretrain-fetch-audit-data``: download (and verify) only the shards an audit interval reads.

    pretrain-fetch-audit-data --checkpoint DIR --gcs-root gs://bucket/shards [--dest ./data/audit_data] [--config-name NAME]
                              [--until-step N] [--no-verify]

``--gcs-root`` (also ``--mirror``) names the mirror of the dataset's shard directory: a ``gs://`` URL or a local directory
with the same layout. The interval runs from the checkpoint's step to ``--until-step`` (default: one checkpoint interval).
Prints what was fetched and the replay command for it. (flags: reference src/pretrain/cli/fetch_audit_data.py:29-62;
mechanics: data/fetch_interval.py)
"""
from __future__ import annotations

import argparse
import json
import logging
import sys


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    ap = argparse.ArgumentParser(prog="pretrain-fetch-audit-data")
    ap.add_argument("--checkpoint", required=True, help="auditable checkpoint directory to start from")
    ap.add_argument("--gcs-root", "--mirror", dest="mirror", required=True, help="gs:// root (or a local directory) holding one <source>/ per source")
    ap.add_argument("--dest", default="./data/audit_data", help="local destination root (default: ./data/audit_data)")
    ap.add_argument("--config-name", default=None, help="train config name (default: the configuration in the checkpoint's meta.json)")
    ap.add_argument("--until-step", type=int, default=None, help="fetch through this optimizer step (default: one checkpoint interval)")
    ap.add_argument("--no-verify", action="store_true", help="skip the blake2b verification of downloaded .idx / .bin files")
    ap.add_argument("--from-init", action="store_true", help="fetch for `pretrain-audit-replay --from-init`: walk from the stream's origin "
                                                             "to --until-step (default: the checkpoint's step)")
    a = ap.parse_args(argv)
    import dataclasses

    from ..data.fetch_interval import fetch_audit_interval

    r = fetch_audit_interval(a.checkpoint, a.mirror, a.dest, until_step=a.until_step, config_name=a.config_name, from_init=a.from_init,
                             verify=not a.no_verify)
    out = dataclasses.asdict(r)
    out.update(checkpoint=a.checkpoint, from_step=r.start_step)
    print(json.dumps(out, indent=2))
    print("\nAudit this interval with:\n  pretrain-audit-replay \\\n      --checkpoint %s \\\n      --data-root %s \\\n%s"
          "      --until-step %d \\\n      --expect-hash <target-checkpoint>/state_hash.txt"
          % (a.checkpoint, r.data_root, "      --from-init \\\n" if a.from_init else "", r.until_step))
    return 0


if __name__ == "__main__":
    sys.exit(main())
