"""``pretrain-eval-olmes``: multiple-choice evaluation of a checkpoint over one or more JSONL task files
({"context", "choices", "answer"} per line; the task is named after the file) through the HF-style wrapper.

Prints one JSON line {"tasks": {name: {"accuracy", "accuracy_raw", "n"}}, "macro": mean accuracy, "step"}; with
``--run-dir`` the same object is also written to ``<run-dir>/evals_olmes/step_<N>/summary.json``, which is what
``scripts/plot_evals_olmes.py`` reads. ``accuracy`` scores a choice by its mean token log-probability, ``accuracy_raw``
by the summed one (the two OLMES normalisations; reference src/pretrain/cli/eval_olmes.py, src/pretrain/eval/olmes_runner.py).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-eval-olmes")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--task-file", required=True, nargs="+")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--limit", type=int)
    ap.add_argument("--run-dir", help="write evals_olmes/step_<N>/summary.json under this run directory")
    a = ap.parse_args(argv)
    from ..data.tokenizer import Tokenizer
    from ..eval.olmes_runner import HFStyleModel, score_multiple_choice
    from .eval import load_model_from_checkpoint

    from ..train.checkpoint import Checkpointer

    model, _cfg, _eng = load_model_from_checkpoint(a.checkpoint, a.device)
    meta = Checkpointer.read_meta(a.checkpoint)
    hf = HFStyleModel(model, Tokenizer(a.tokenizer))
    tasks = {}
    for tf in a.task_file:
        rows = [json.loads(l) for l in Path(tf).read_text().splitlines() if l.strip()][: a.limit]
        hit = {"per_token": 0, "sum": 0}
        for r in rows:
            for norm in hit:
                hit[norm] += score_multiple_choice(hf, r["context"], r["choices"], norm)["prediction"] == r["answer"]
        n = max(len(rows), 1)
        tasks[Path(tf).stem] = {"accuracy": hit["per_token"] / n, "accuracy_raw": hit["sum"] / n, "n": len(rows)}
    step = int(getattr(meta, "step", 0) or 0)
    out = {"step": step, "consumed_tokens": int(getattr(meta, "consumed_tokens", 0) or 0), "tasks": tasks,
           "macro": sum(t["accuracy"] for t in tasks.values()) / max(len(tasks), 1)}
    if a.run_dir:
        d = Path(a.run_dir) / "evals_olmes" / ("step_%09d" % step)
        d.mkdir(parents=True, exist_ok=True)
        (d / "summary.json").write_text(json.dumps(out, indent=1) + "\n")
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
