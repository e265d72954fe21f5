"""One micro-batch of the CPU replay at a recipe's full size: forward + backward of `micro_batch_size x seq_len` tokens through
the C++ twins, wall time and peak resident set. A step of the replay is `microbatches per step` of these plus the reduction
and AdamW, so this is the unit that sizes a CPU audit.

    python benchmarks/cpu_microbatch.py --config-name open1b_b200 --override run.activation_checkpoint=true

The engine is built the way the replay builds it (one work buffer for the gradients, moments in files); the tokens are random
(the time does not depend on them). Prints two JSON lines: after the engine is built, and after the micro-batch.
"""
from __future__ import annotations

import argparse
import json
import os
import resource
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rss_gb() -> float:
    return round(resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 2 ** 20, 1)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-name", default="open1b_b200")
    ap.add_argument("--override", nargs="*", default=[])
    ap.add_argument("--cpu-threads", default="auto")
    ap.add_argument("--keep-moments-in-memory", action="store_true", help="do not put the AdamW moments in files (needs 8 bytes per parameter more)")
    a = ap.parse_args()
    import torch

    from open_transformers_b200.cli.cpu_threads import configure_cpu_threads
    from open_transformers_b200.config import load_config
    from open_transformers_b200.train.engine import TrainEngine

    threads = configure_cpu_threads(a.cpu_threads)
    cfg = load_config(a.config_name, list(a.override))
    t0 = time.time()
    with tempfile.TemporaryDirectory() as off:
        eng = TrainEngine(cfg, "cpu", 0, 1, init=True, fold_gradients=True, offload_optimizer=not a.keep_moments_in_memory,
                          optimizer_offload_dir=off)
        print(json.dumps({"engine_s": round(time.time() - t0, 1), "rss_gb": rss_gb(), "threads": threads}), flush=True)
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(0, cfg.model.vocab_size, (cfg.train.micro_batch_size, cfg.train.seq_len), generator=g)
        t1 = time.time()
        out = eng.forward_backward(0, ids, torch.roll(ids, -1, 1), 1, last=True)
        dt = time.time() - t1
        print(json.dumps({"microbatch_fwd_bwd_s": round(dt, 1), "tokens": ids.numel(), "tokens_per_s": round(ids.numel() / dt, 2),
                          "loss_ce": float(out[0].detach()), "loss_z": float(out[1].detach()), "peak_rss_gb": rss_gb()}), flush=True)
        eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
