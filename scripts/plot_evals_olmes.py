#!/usr/bin/env python
"""Plot multiple-choice (OLMES-style) evaluation results of one or more run directories against the training step.

    python scripts/plot_evals_olmes.py runs/<RUN_ID>
    python scripts/plot_evals_olmes.py runs/<a> runs/<b> --labels baseline candidate -o olmes.png
    python scripts/plot_evals_olmes.py runs/<a> runs/<a-resumed> --stitch

Reads every ``<run>/evals_olmes/step_<N>/summary.json`` written by ``pretrain-eval-olmes --run-dir`` ({"step", "tasks":
{name: {"accuracy", "accuracy_raw", "n"}}, "macro"}) and draws the macro average plus one panel per task: the
per-token-normalised accuracy as a solid line and the raw (summed log-probability) accuracy dashed, since which of
the two formulations wins is itself informative for small models. ``--stitch`` joins several directories (a run and its
resumed continuations) into one trace, later directories winning on equal steps. Without matplotlib the points are
printed as CSV. (reference scripts/plot_evals_olmes.py)
"""
import argparse
import json
import sys
from pathlib import Path


def load_run(run_dir: Path) -> dict:
    """{step: summary} of one run directory."""
    out = {}
    for f in sorted((run_dir / "evals_olmes").glob("step_*/summary.json")):
        s = json.loads(f.read_text())
        out[int(s.get("step", int(f.parent.name.split("_")[1])))] = s
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--labels", nargs="*")
    ap.add_argument("--stitch", action="store_true", help="treat all directories as segments of one run")
    ap.add_argument("-o", "--output", "--out", dest="out", default="evals_olmes.png")
    ap.add_argument("--best-only", action="store_true", help="only the headline score per task (no dashed raw-accuracy trace)")
    a = ap.parse_args(argv)
    runs = [(Path(r), load_run(Path(r))) for r in a.runs]
    if a.stitch:
        merged = {}
        for _, pts in runs:
            merged.update(pts)
        runs = [(runs[0][0], merged)]
    labels = a.labels if a.labels and len(a.labels) == len(runs) else [r.name for r, _ in runs]
    tasks = sorted({t for _, pts in runs for s in pts.values() for t in s["tasks"]})
    if not any(pts for _, pts in runs):
        print("no evals_olmes/step_*/summary.json under", ", ".join(a.runs), file=sys.stderr)
        return 1
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        print("run,step,series,value")
        for label, (_, pts) in zip(labels, runs):
            for step in sorted(pts):
                print("%s,%d,macro,%.6f" % (label, step, pts[step]["macro"]))
                for t, v in pts[step]["tasks"].items():
                    print("%s,%d,%s,%.6f" % (label, step, t, v["accuracy"]))
                    if not a.best_only:
                        print("%s,%d,%s_raw,%.6f" % (label, step, t, v["accuracy_raw"]))
        return 0
    n = 1 + len(tasks)
    cols = min(3, n)
    rows_ = (n + cols - 1) // cols
    fig, axes = plt.subplots(rows_, cols, figsize=(5 * cols, 3.2 * rows_), squeeze=False)
    flat = axes.ravel()
    for label, (_, pts) in zip(labels, runs):
        steps = sorted(pts)
        flat[0].plot(steps, [pts[s]["macro"] for s in steps], marker="o", label=label)
        for ax, t in zip(flat[1:], tasks):
            have = [s for s in steps if t in pts[s]["tasks"]]
            line, = ax.plot(have, [pts[s]["tasks"][t]["accuracy"] for s in have], marker="o", label=label)
            if not a.best_only:
                ax.plot(have, [pts[s]["tasks"][t]["accuracy_raw"] for s in have], linestyle="--", color=line.get_color())
    flat[0].set_title("macro average")
    for ax, t in zip(flat[1:], tasks):
        ax.set_title(t)
    for ax in flat[:n]:
        ax.set_xlabel("step")
        ax.set_ylabel("accuracy")
        ax.grid(alpha=0.3)
    for ax in flat[n:]:
        ax.axis("off")
    flat[0].legend()
    fig.tight_layout()
    fig.savefig(a.out, dpi=120)
    print("wrote", a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
