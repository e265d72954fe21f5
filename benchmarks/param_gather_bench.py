"""Parameter all-gather fused into the consuming GEMM (`otb_pg_gemm`) against the library way (NCCL all-gather of the
weight rows into a full buffer, then the plain GEMM), one node, N GPUs, launched with torch.distributed.run:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
      benchmarks/param_gather_bench.py --tokens 16384

For the four projection shapes of the OPEN-1B block and the vocabulary head it reports, per shape: the plain GEMM on a
complete weight (no communication: the floor), the fused call (every call pulls the (P-1)/P foreign rows again: the flag
value changes per call), and all-gather + GEMM; times are CUDA events on the launching stream, max over ranks, inputs
rotated through buffers larger than L2. The roofline of the fused call is the slower of FLOPs / measured GEMM rate and
pulled bytes / 770 GB/s. With one process (`python benchmarks/param_gather_bench.py --emulate 4`) the owners are buffers
of the same GPU: the pull is then local HBM traffic, which times the kernel's structure but not NVLink.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.ops import functional as K
from open_transformers_b200.parallel.flat import PeerBuffer
from open_transformers_b200.parallel.param_gather import GatheredWeight, flag_words

NVLINK_PEER_GBS = 770.0
SHAPES = [("qkv", [2048, 512, 512], 2048), ("attn_out", [2048], 2048), ("gate_up", [11264], 2048), ("down", [2048], 5632),
          ("vocab_head", [128256], 2048)]


def timed(fn, iters, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--emulate", type=int, default=0, help="single process: this many owners as buffers of the one GPU")
    ap.add_argument("--gemm-tflops", type=float, default=1400.0, help="measured sustained bf16 GEMM rate for the roofline")
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    P = world if world > 1 else max(1, a.emulate)
    me = rank if world > 1 else 0
    M = a.tokens
    g = torch.Generator().manual_seed(1)
    rows = []
    for name, seg_rows, Kd in SHAPES:
        N = sum(seg_rows)
        W = (0.02 * torch.randn(N, Kd, generator=g)).bfloat16().to(dev)
        xs = [torch.randn(M, Kd, generator=g).bfloat16().to(dev) for _ in range(3)]   # rotated: 3 x 64 MB and the weight exceed L2 together
        seg_begin = [sum(seg_rows[:j]) for j in range(len(seg_rows))]
        rpo = [-(-r // P) for r in seg_rows]
        if world > 1:
            buf = PeerBuffer(W.numel() * 2, dev, rank, world)
            local_w = buf.typed(torch.bfloat16).view(N, Kd)
            ptrs = list(buf.ptrs)
        else:
            bufs = [torch.empty_like(W) for _ in range(P)]
            local_w, ptrs = bufs[0], [b.data_ptr() for b in bufs]
            for b in bufs:
                b.copy_(W)
        local_w.copy_(W)
        flags = torch.zeros(flag_words(N), dtype=torch.int32, device=dev)
        gw = GatheredWeight(local_w, ptrs, me, seg_begin, rpo, flags)
        state = {"i": 0}

        def plain():
            state["i"] += 1
            K.gemm(xs[state["i"] % 3], local_w)

        def fused():
            state["i"] += 1
            gw.epoch += 1
            gw.gemm(xs[state["i"] % 3])

        # library way: every process contributes its rows (the first weight's split stands for all of them), then the GEMM
        shard = torch.empty((-(-N // P), Kd), dtype=torch.bfloat16, device=dev)
        full = torch.empty((P * shard.shape[0], Kd), dtype=torch.bfloat16, device=dev)

        def library():
            state["i"] += 1
            if world > 1:
                dist.all_gather_into_tensor(full, shard)
            K.gemm(xs[state["i"] % 3], full[:N])

        # fused first, plain before and after it: a difference between the two plain figures is clock drift under the power cap
        t_plain0 = timed(plain, a.iters, world)
        t_fused = timed(fused, a.iters, world)
        t_plain = timed(plain, a.iters, world)
        t_lib = timed(library, a.iters, world) if world > 1 else None
        ok = bool(torch.equal(gw.gemm(xs[0]).view(torch.int16), K.gemm(xs[0], W).view(torch.int16)))
        flops = 2.0 * M * N * Kd
        pulled = 2.0 * N * Kd * (P - 1) / P
        roof_ms = max(flops / (a.gemm_tflops * 1e12), pulled / (NVLINK_PEER_GBS * 1e9)) * 1e3
        rows.append({"shape": name, "M": M, "N": N, "K": Kd, "owners": P, "plain_ms": t_plain, "plain_before_ms": t_plain0, "fused_ms": t_fused, "allgather_gemm_ms": t_lib,
                     "pulled_mb": pulled / 1e6, "roofline_ms": roof_ms, "fused_of_roofline": roof_ms / t_fused, "same_bits": ok})
        del gw, local_w, W, xs, full, shard
        if world > 1:
            dist.barrier()
            buf.close()
        torch.cuda.empty_cache()
    status = K.kernel_status(dev)
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"kernel_status": status, "emulated_owners": a.emulate if world == 1 else 0}))
    if world > 1:
        dist.destroy_process_group()
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
