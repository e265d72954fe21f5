"""Where one optimizer step spends its device time, per native entry point, on one B200.

  python benchmarks/step_breakdown.py [--config open1b_b200] [--microbatches 2] [--override k=v ...]

Runs one warm-up micro-batch, then traces ``--microbatches`` forward+backward passes, the gradient reduction,
the AdamW step and the state hash with the CUDA-event tracer of ``ops/native.py`` (one event after every native
call, resolved after the end). PyTorch ops between two native calls are charged to the later call. Prints a table
sorted by time and one JSON line. The figures are shares for finding the next kernel to work on; the step time
that counts is bench.py's.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from open_transformers_b200.config import load_config
from open_transformers_b200.ops import native
from open_transformers_b200.train.engine import TrainEngine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="open1b_b200")
    ap.add_argument("--microbatches", type=int, default=2)
    ap.add_argument("--override", action="append", default=[])
    args = ap.parse_args()
    cfg = load_config(args.config, args.override)
    dev = torch.device("cuda", 0)
    native.cuda_lib()
    eng = TrainEngine(cfg, dev)
    mb, T, vocab = cfg.train.micro_batch_size, cfg.train.seq_len, cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)

    def batch():
        seq = torch.randint(0, vocab, (mb, T + 1), generator=g)
        return seq[:, :-1].contiguous().to(dev), seq[:, 1:].contiguous().to(dev)

    batches = [batch() for _ in range(args.microbatches + 1)]
    eng.zero_grads()
    eng.forward_backward(0, *batches[0], 1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    native.start_timing()
    native.mark("start")
    e0.record()
    for ids, labels in batches[1:]:
        eng.forward_backward(0, ids, labels, 1)
        native.mark("torch: loss + autograd tail")
    norm = eng.reduce_gradients()
    native.mark("torch: norm fold (host)")
    eng.optimizer_step(3e-4, eng.clip_coefficient(norm, cfg.train.grad_clip))
    eng.sharded_state_hash(None, None, include_grads=cfg.train.state_hash.include_grads)
    native.mark("state hash (tree digests + host combine)")
    e1.record()
    rep = native.timing_report()
    total = e0.elapsed_time(e1)
    rows = sorted(rep.items(), key=lambda kv: -kv[1][1])
    print("%-52s %6s %10s %7s" % ("entry point", "calls", "ms", "share"))
    for what, (n, ms) in rows:
        print("%-52s %6d %10.3f %6.1f%%" % (what, n, ms, 100.0 * ms / total))
    print("%-52s %6s %10.3f" % ("total (events)", "", total))
    print(json.dumps({"total_ms": total, "microbatches": args.microbatches,
                      "rows": {k: {"calls": n, "ms": ms} for k, (n, ms) in rows}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
