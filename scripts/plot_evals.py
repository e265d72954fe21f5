#!/usr/bin/env python
"""Plot the DCLM-CORE evaluation results of one or more run directories against the training step.

    python scripts/plot_evals.py runs/<RUN_ID>
    python scripts/plot_evals.py runs/<a> runs/<b> --labels baseline candidate
    python scripts/plot_evals.py runs/<a> -o evals.png
    python scripts/plot_evals.py runs/<a> runs/<a-resumed> --stitch

Reads every ``<run>/evals/step_<N>/step_*.json`` that ``pretrain-eval --out-dir <run>/evals/step_<N>`` wrote ({"step",
"tasks": {name: {"primary", ...}}, "categories", "category_tasks", "macro_average"}) and draws the overall macro average,
one panel per category (a category with a single task carries the task's name) and one panel per task. ``--stitch`` treats
the directories as consecutive segments of one resumed run, given in order; where two segments evaluated the same step
the later one wins. Without matplotlib the points are printed as CSV. (same command line as the reference's
scripts/plot_evals.py; training curves from ``logs/metrics.jsonl`` are ``scripts/plot_training_curves.py``)
"""
import argparse
import json
import sys
from pathlib import Path

CATEGORY, TASK = "cat:", "task:"


def load_run(run_dir: Path):
    """(points sorted by step, {category: set of task names}) of one run directory; a point is {"step", "macro",
    "cat:<name>", "task:<name>"}."""
    evals = run_dir / "evals"
    if not evals.exists():
        raise SystemExit("no evals directory at %s" % evals)
    points, members = [], {}
    for d in sorted(evals.glob("step_*")):
        files = sorted(d.glob("step_*.json")) if d.is_dir() else []
        if not files:
            continue
        result = json.loads(files[0].read_text())
        point = {"step": int(d.name[len("step_"):]), "macro": result.get("macro_average")}
        for name, value in (result.get("categories") or {}).items():
            point[CATEGORY + name] = value
        for name, info in (result.get("tasks") or {}).items():
            if isinstance(info, dict) and info.get("primary") is not None:
                point[TASK + name] = info["primary"]
        points.append(point)
        for name, tasks in (result.get("category_tasks") or {}).items():
            members.setdefault(name, set()).update(tasks)
    if not points:
        raise SystemExit("no eval results found under %s" % evals)
    return sorted(points, key=lambda p: p["step"]), members


def stitch(segments):
    """One series from the segments of a resumed run: by step, later segments overwrite earlier ones."""
    by_step = {}
    for points in segments:
        for p in points:
            by_step[p["step"]] = p
    return [by_step[s] for s in sorted(by_step)]


def single_task_of(points, category: str):
    """For results without ``category_tasks``: the one task whose score equals the category's at every step, if any (an
    average over several tasks practically never coincides with one member)."""
    candidates = None
    for p in points:
        if CATEGORY + category not in p:
            continue
        here = {k[len(TASK):] for k in p if k.startswith(TASK) and p[k] == p[CATEGORY + category]}
        candidates = here if candidates is None else candidates & here
    return next(iter(candidates)) if candidates and len(candidates) == 1 else None


def layout(series, members_per_run):
    """[(point key, panel title)]: macro, categories (single-task ones under the task's name), then tasks not shown yet."""
    keys = []
    for _label, points in series:
        for p in points:
            for k in p:
                if k not in ("step", "macro") and k not in keys:
                    keys.append(k)
    panels, shown = [("macro", "macro average")], set()
    for k in [k for k in keys if k.startswith(CATEGORY)]:
        name = k[len(CATEGORY):]
        tasks = set()
        for members in members_per_run:
            tasks |= members.get(name, set())
        only = next(iter(tasks)) if len(tasks) == 1 else (single_task_of([p for _l, pts in series for p in pts], name) if not tasks else None)
        panels.append((k, only or name))
        if only:
            shown.add(only)
    for k in [k for k in keys if k.startswith(TASK)]:
        if k[len(TASK):] not in shown:
            panels.append((k, k[len(TASK):]))
    return panels


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--labels", nargs="*")
    ap.add_argument("--stitch", action="store_true", help="the directories are consecutive segments of one resumed run")
    ap.add_argument("-o", "--output", "--out", dest="out", default="evals.png")
    a = ap.parse_args(argv)
    loaded = [load_run(Path(r)) for r in a.runs]
    members = [m for _p, m in loaded]
    if a.stitch:
        series = [((a.labels or [Path(a.runs[0]).name])[0], stitch([p for p, _m in loaded]))]
    else:
        labels = a.labels if a.labels and len(a.labels) == len(a.runs) else [Path(r).name for r in a.runs]
        series = [(label, points) for label, (points, _m) in zip(labels, loaded)]
    panels = layout(series, members)
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        print("run,step," + ",".join(title for _k, title in panels))
        for label, points in series:
            for p in points:
                print(",".join([label, str(p["step"])] + ["" if p.get(k) is None else "%.6g" % p[k] for k, _t in panels]))
        return 0
    cols = min(3, len(panels))
    rows = -(-len(panels) // cols)
    fig, axes = plt.subplots(rows, cols, figsize=(5 * cols, 3.2 * rows), squeeze=False)
    for ax, (key, title) in zip(axes.flat, panels):
        for label, points in series:
            xs = [p["step"] for p in points if p.get(key) is not None]
            ax.plot(xs, [p[key] for p in points if p.get(key) is not None], marker="o", markersize=3, label=label)
        ax.set_title(title)
        ax.set_xlabel("step")
        ax.grid(alpha=0.3)
    for ax in list(axes.flat)[len(panels):]:
        ax.set_visible(False)
    axes.flat[0].legend()
    fig.tight_layout()
    fig.savefig(a.out, dpi=120)
    print("wrote %s" % a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
