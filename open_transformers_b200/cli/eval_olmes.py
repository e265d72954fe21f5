"""``pretrain-eval-olmes``: multiple-choice evaluation of a checkpoint over a JSONL task file
({"context", "choices", "answer"} per line) through the HF-style wrapper."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-eval-olmes")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--task-file", required=True)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--limit", type=int)
    a = ap.parse_args(argv)
    from ..data.tokenizer import Tokenizer
    from ..eval.olmes_runner import HFStyleModel, score_multiple_choice
    from .eval import load_model_from_checkpoint

    model, _, _ = load_model_from_checkpoint(a.checkpoint, a.device)
    hf = HFStyleModel(model, Tokenizer(a.tokenizer))
    rows = [json.loads(l) for l in Path(a.task_file).read_text().splitlines() if l.strip()][: a.limit]
    correct = sum(score_multiple_choice(hf, r["context"], r["choices"])["prediction"] == r["answer"] for r in rows)
    print(json.dumps({"accuracy": correct / max(len(rows), 1), "n": len(rows)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
