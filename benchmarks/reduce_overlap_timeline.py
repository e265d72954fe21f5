"""When each bucket of gradients enters and leaves the reduction, relative to the backward pass that produces it.

  python benchmarks/reduce_overlap_timeline.py                                   # one GPU
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
         benchmarks/reduce_overlap_timeline.py [--steps 4] [--config open1b_b200]

Runs `--steps` optimizer steps of the recipe with OTB_REDUCE_TIMELINE=1 and prints, for the last step on rank 0, one
row per bucket (vocabulary head, blocks last to first, embedding): when the backward pass had finished it, when its
reduction started (every rank had signalled the bucket) and ended, all in ms after the first bucket was ready, and the
end of the backward pass on the same clock. A reduction that ends before `backward end` cost the step nothing.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

os.environ["OTB_REDUCE_TIMELINE"] = "1"
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.config import load_config
from open_transformers_b200.ops import native
from open_transformers_b200.train.engine import TrainEngine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="open1b_b200")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--override", action="append", default=[])
    args = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    native.cuda_lib()
    cfg = load_config(args.config, args.override)
    eng = TrainEngine(cfg, dev, rank, world, None)
    V, mb, T, vocab = cfg.run.virtual_dp_size, cfg.train.micro_batch_size, cfg.train.seq_len, cfg.model.vocab_size
    accum = max(1, cfg.train.global_batch_tokens.main // (mb * T * V))
    hosted = eng.hosted
    rows = []
    for step in range(args.steps):
        eng.zero_grads()
        for vi, v in enumerate(hosted):
            for k in range(accum):
                g = torch.Generator().manual_seed((step * V + v) * accum + k)
                seq = torch.randint(0, vocab, (mb, T + 1), generator=g)
                eng.forward_backward(vi, seq[:, :-1].contiguous().to(dev), seq[:, 1:].contiguous().to(dev), accum,
                                     last=(vi == len(hosted) - 1 and k == accum - 1))
        t = eng.overlap_timeline()
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, cfg.train.grad_clip))
        rows = t or rows
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if rank == 0:
        print("| bucket | chunks owned | ready (ms) | reduction start (ms) | reduction end (ms) |")
        print("|---|---|---|---|---|")
        L = cfg.model.n_layers
        for r in rows:
            b = r["bucket"]
            name = "head" if b == 0 else ("embedding" if b == L + 1 else "block %d%s" % (L - b, " + final norm" if b == 1 else ""))
            print("| %s | %d | %.2f | %.2f | %.2f |" % (name, r["chunks"], r["ready_ms"], r["reduce_start_ms"], r["reduce_end_ms"]))
        if rows:
            print("backward end: %.2f ms; last reduction end: %.2f ms; GPUs: %d" % (rows[0].get("backward_end_ms", float("nan")),
                                                                                   max(r["reduce_end_ms"] for r in rows), world))
        print(json.dumps({"world": world, "rows": rows}))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
