"""``pretrain-eval-olmes``: OLMES evaluation of a checkpoint.

    pretrain-eval-olmes --checkpoint CKPT --tokenizer tokenizer.json --out-dir DIR [--task NAME ...] [--extended]
                        [--batch-size 4] [--max-length 2048] [--limit N] [--model-label L]          (needs oe_eval + lm_eval)
    pretrain-eval-olmes --checkpoint CKPT --tokenizer tokenizer.json --task-file a.jsonl b.jsonl [--limit N] [--run-dir RUN]

The first form runs the OLMES suites through AllenAI's ``oe_eval`` (default suites ``core_9mcqa::olmes`` and
``mmlu::olmes``; ``--extended`` adds the generative extension tasks) and prints ``summary.json`` (reference
src/pretrain/cli/eval_olmes.py, src/pretrain/eval/olmes_runner.py:292-398). The second needs no extra package: it scores
multiple-choice JSONL task files ({"context", "choices", "answer"} per line; a task is named after its file) and prints
{"tasks": {name: {"accuracy", "accuracy_raw", "n"}}, "macro", "step"}; with ``--run-dir`` the object is also written to
``<run-dir>/evals_olmes/step_<N>/summary.json``, which ``scripts/plot_evals_olmes.py`` reads. The model configuration
comes from the checkpoint's ``meta.json``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    from ..eval.olmes_runner import OLMES_DEFAULT_SUITES, OLMES_MAX_LENGTH

    ap = argparse.ArgumentParser(prog="pretrain-eval-olmes")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--config-name", default=None, help="train config name (default: the configuration recorded in the checkpoint)")
    ap.add_argument("--override", nargs="*", default=[], help="config overrides (with --config-name)")
    ap.add_argument("--out-dir", help="oe_eval output directory (metrics-all.jsonl, predictions, summary.json)")
    ap.add_argument("--task", nargs="*", default=None, help="olmes task / suite names (default: %s)" % " ".join(OLMES_DEFAULT_SUITES))
    ap.add_argument("--extended", action="store_true", help="also the generative extension tasks (hours at 1 B parameters)")
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--max-length", type=int, default=OLMES_MAX_LENGTH)
    ap.add_argument("--model-label", default=None)
    ap.add_argument("--task-file", nargs="+", help="score these multiple-choice JSONL files with the built-in scorer instead")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--limit", type=int, help="cap the instances per task (smoke runs; breaks comparability)")
    ap.add_argument("--run-dir", help="built-in scorer: write evals_olmes/step_<N>/summary.json under this run directory")
    a = ap.parse_args(argv)
    from ..eval import olmes_runner as R
    from ..train.checkpoint import Checkpointer
    from .eval import load_model_from_checkpoint

    if not a.task_file and not a.out_dir:
        ap.error("give --out-dir (oe_eval suites) or --task-file (built-in scorer)")
    if not a.task_file and not R.olmes_available():
        print("pretrain-eval-olmes: the OLMES suites need the oe_eval and lm_eval packages, which are not installed; "
              "use --task-file with local JSONL tasks", file=sys.stderr)
        return 2
    model, _cfg, _eng = load_model_from_checkpoint(a.checkpoint, a.device, config_name=a.config_name, overrides=a.override)
    meta = Checkpointer.read_meta(a.checkpoint)
    if not a.task_file:
        out = R.run_olmes(model, a.tokenizer, a.out_dir, tasks=a.task, extended=a.extended, batch_size=a.batch_size, max_length=a.max_length,
                          limit=a.limit, device=a.device, model_label=a.model_label or Path(a.checkpoint).name)
        print(json.dumps(out, indent=2))
        return 0
    from ..data.tokenizer import Tokenizer

    tasks = R.run_task_files(R.HFStyleModel(model, Tokenizer(a.tokenizer)), a.task_file, a.limit)
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
