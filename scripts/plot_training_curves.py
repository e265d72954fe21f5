#!/usr/bin/env python
"""Plot loss / grad-norm / throughput curves from one or more runs' logs/metrics.jsonl (matplotlib if present,
otherwise a CSV dump)."""
import argparse
import json
from pathlib import Path


def load(path):
    return [json.loads(l) for l in Path(path).read_text().splitlines() if l.strip()]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("metrics", nargs="+")
    ap.add_argument("--keys", default="loss,grad_norm_pre_clip,tokens_per_sec")
    ap.add_argument("--out", default="curves.png")
    a = ap.parse_args()
    keys = a.keys.split(",")
    runs = {p: load(p) for p in a.metrics}
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        for p, rows in runs.items():
            for r in rows:
                print(",".join([p, str(r.get("step"))] + [str(r.get(k)) for k in keys]))
        return
    fig, axes = plt.subplots(len(keys), 1, figsize=(8, 3 * len(keys)), squeeze=False)
    for ax, k in zip(axes[:, 0], keys):
        for p, rows in runs.items():
            ax.plot([r["consumed_tokens"] for r in rows], [r.get(k) for r in rows], label=Path(p).parent.parent.name)
        ax.set_ylabel(k)
        ax.legend()
    axes[-1, 0].set_xlabel("consumed tokens")
    fig.savefig(a.out, dpi=120)


if __name__ == "__main__":
    main()
