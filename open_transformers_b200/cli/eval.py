"""``pretrain-eval --checkpoint DIR --tokens FILE.bin|prefix``: held-out perplexity (and, given task accuracies,
the DCLM-CORE aggregate)."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def load_model_from_checkpoint(checkpoint: str, device: str = "cpu"):
    from ..config import parse_config_resolved
    from ..train.checkpoint import Checkpointer
    from ..train.engine import TrainEngine

    meta = Checkpointer.read_meta(checkpoint)
    cfg = parse_config_resolved(meta.config_resolved)
    cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size, cfg.run.tp_size = 1, 1, 1, 1
    eng = TrainEngine(cfg, device, 0, 1, init=False)
    Checkpointer(Path(checkpoint).parent.parent).load(checkpoint, eng, load_optimizer=False)
    eng._bind_slots(None)
    return eng.model, cfg, eng


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-eval")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--shard-prefix", required=True, help="held-out .bin/.idx shard prefix")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--max-tokens", type=int, default=1 << 20)
    ap.add_argument("--stride", type=int)
    ap.add_argument("--batch-windows", type=int, default=8, help="windows of equal length scored per forward pass")
    ap.add_argument("--task-accuracies", help="JSON file {task: accuracy} for the DCLM-CORE aggregate")
    a = ap.parse_args(argv)
    import numpy as np
    import torch

    from ..data.indexed_dataset import IndexedDatasetReader
    from ..eval.dclm_core import dclm_core_score
    from ..eval.perplexity import perplexity

    model, cfg, _ = load_model_from_checkpoint(a.checkpoint, a.device)
    r = IndexedDatasetReader(a.shard_prefix)
    toks = np.concatenate([np.asarray(r.document(i), dtype=np.int64) for i in range(r.num_documents)])[: a.max_tokens]
    out = {"perplexity": perplexity(model, torch.from_numpy(toks), cfg.train.seq_len, a.stride, a.batch_windows), "tokens": int(len(toks))}
    if a.task_accuracies:
        out["dclm_core"] = dclm_core_score(json.loads(Path(a.task_accuracies).read_text()))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
