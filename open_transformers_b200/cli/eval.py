"""``pretrain-eval --checkpoint DIR --tokenizer tokenizer.json --out-dir DIR [--held-out PREFIX] [--no-dclm] [--config-name NAME
[--override ...]]``: held-out perplexity and the DCLM-CORE slice of a checkpoint."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def load_model_from_checkpoint(checkpoint: str, device: str = "cpu", config_name: str | None = None, overrides=None):
    """(model, cfg, engine) of a checkpoint on one device. The configuration is the one the checkpoint recorded unless a
    config name (with overrides) is given."""
    from ..config import load_config, parse_config_resolved
    from ..train.checkpoint import Checkpointer
    from ..train.engine import TrainEngine

    meta = Checkpointer.read_meta(checkpoint)
    cfg = load_config(config_name, list(overrides or [])) if config_name else parse_config_resolved(meta.config_resolved)
    cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size, cfg.run.tp_size = 1, 1, 1, 1
    eng = TrainEngine(cfg, device, 0, 1, init=False)
    Checkpointer(Path(checkpoint).parent.parent).load(checkpoint, eng, load_optimizer=False)
    eng._bind_slots(None)
    return eng.model, cfg, eng


def main(argv=None) -> int:
    """Flags as the reference's tool has them (src/pretrain/cli/eval.py:26-86): held-out perplexity with ``--held-out``, the
    DCLM-CORE slice unless ``--no-dclm``; ``<out-dir>/summary.json`` and the same object on stdout. The model configuration
    comes from the checkpoint's ``meta.json`` (``--config-name`` / ``--override`` replace it when given)."""
    ap = argparse.ArgumentParser(prog="pretrain-eval")
    ap.add_argument("--config-name", default=None, help="train config name (default: the configuration recorded in the checkpoint)")
    ap.add_argument("--checkpoint", required=True, help="checkpoint directory to load")
    ap.add_argument("--tokenizer", default=None, help="tokenizer.json (needed for the DCLM-CORE tasks)")
    ap.add_argument("--held-out", "--shard-prefix", dest="held_out", help="held-out .bin/.idx shard prefix for the perplexity")
    ap.add_argument("--out-dir", default=None, help="where summary.json and the DCLM-CORE result file go")
    ap.add_argument("--no-dclm", action="store_true", help="skip the DCLM-CORE run")
    ap.add_argument("--override", nargs="*", default=[], help="config overrides (with --config-name)")
    ap.add_argument("--device", default=None, help="cuda or cpu (default: cuda when there is one)")
    ap.add_argument("--max-tokens", type=int, default=1 << 20, help="held-out tokens scored")
    ap.add_argument("--stride", type=int)
    ap.add_argument("--batch-windows", type=int, default=8, help="windows of equal length scored per forward pass")
    ap.add_argument("--task-accuracies", help="JSON file {task: accuracy}: adds the centred DCLM-CORE aggregate of ready-made accuracies")
    a = ap.parse_args(argv)
    import numpy as np
    import torch

    from ..data.indexed_dataset import IndexedDatasetReader
    from ..eval.dclm_core import dclm_core_score, run_dclm_core
    from ..eval.perplexity import perplexity
    from ..train.checkpoint import Checkpointer

    if not a.no_dclm and not a.tokenizer:
        ap.error("--tokenizer is needed for the DCLM-CORE tasks (or pass --no-dclm)")
    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model, cfg, _ = load_model_from_checkpoint(a.checkpoint, device, config_name=a.config_name, overrides=a.override)
    step = int(getattr(Checkpointer.read_meta(a.checkpoint), "step", 0) or 0)
    out_dir = Path(a.out_dir) if a.out_dir else None
    if out_dir:
        out_dir.mkdir(parents=True, exist_ok=True)
    summary: dict = {}
    if a.held_out:
        r = IndexedDatasetReader(a.held_out)
        toks = np.concatenate([np.asarray(r.document(i), dtype=np.int64) for i in range(r.num_documents)])[: a.max_tokens]
        summary["held_out_ppl"] = perplexity(model, torch.from_numpy(toks), cfg.train.seq_len, a.stride, a.batch_windows)
        summary["held_out_tokens"] = int(len(toks))
    if not a.no_dclm:
        import tempfile

        from ..data.tokenizer import Tokenizer

        result = run_dclm_core(model, Tokenizer(a.tokenizer), out_dir or tempfile.mkdtemp(prefix="dclm_core_"), step, device=device)
        summary["dclm_core_macro"] = result.get("macro_average")
        if "error" in result:
            summary["dclm_core_error"] = result["error"]
    if a.task_accuracies:
        summary["dclm_core"] = dclm_core_score(json.loads(Path(a.task_accuracies).read_text()))
    if out_dir:
        (out_dir / "summary.json").write_text(json.dumps(summary, indent=2))
    print(json.dumps(summary, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
