"""Deterministic gradient-reduction micro-benchmark (one node, N GPUs, launched with torch.distributed.run).

Every rank holds one fp32 gradient bucket per virtual rank it hosts (normal(0, 1e-3), seeded per virtual rank). The
fused kernel reduces each rank's share of the bucket by pulling all S x R buckets over NVLink peer loads in ascending
shard order, x 1/S, binary-blocks tree over R replicas, x 1/R, and emits the squared-norm partials in the same pass.
Reported per message size: time (CUDA events, max over ranks), algorithmic bus bandwidth
    busbw = (bytes pulled from peers per rank) / time
against the measured NVLink peer-copy figure (770 GB/s per direction), and the same reduction done with NCCL
(all_to_all_single of the bucket + local ascending adds = the reference's DeterministicReduceScatter,
src/pretrain/parallel/deterministic_reduce.py:77-117). For sizes up to --verify-mb (default: all of them) every rank
compares its slice of the result, and its squared-norm partials, bit for bit with the CPU twin applied to the same slice of
all S x R buckets (regenerated from their seeds).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
      benchmarks/reduce_bench.py --shard 4 --replicate 2 --sizes-mb 1,16,256,1024
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.ops.native import I, P, check, cpu_lib, cuda_lib, stream_ptr
from open_transformers_b200.parallel.flat import CHUNK, PeerBuffer

NVLINK_PEER_GBS = 770.0


def ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shard", type=int, default=0, help="virtual shard-group size S (default: number of GPUs)")
    ap.add_argument("--replicate", type=int, default=1)
    ap.add_argument("--sizes-mb", default="1,4,16,64,256,1024")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--verify-mb", type=float, default=1024, help="check the result bit for bit against the CPU fold up to this bucket size")
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    S = a.shard or world
    R = a.replicate
    V = S * R
    assert V % world == 0, "virtual ranks must split evenly over the GPUs"
    per = V // world
    lib = cuda_lib()
    rows = []
    for mb in [float(x) for x in a.sizes_mb.split(",")]:
        n = int(mb * (1 << 20) / 4) // (CHUNK * world) * (CHUNK * world)
        n = max(n, CHUNK * world)
        bufs = [PeerBuffer(4 * n, dev, rank, world) for _ in range(per)]
        for slot, b in enumerate(bufs):
            v = rank * per + slot
            g = torch.Generator(device=dev).manual_seed(1234 + v)
            b.typed(torch.float32).copy_(torch.randn(n, device=dev, generator=g) * 1e-3)
        out = torch.zeros(n, dtype=torch.float32, device=dev)
        n_chunks = n // CHUNK
        own = n_chunks // world
        cs = torch.arange(rank * own, (rank + 1) * own, device=dev, dtype=torch.int64) * CHUNK
        cl = torch.full((own,), CHUNK, dtype=torch.int32, device=dev)
        sos = torch.zeros(own, dtype=torch.float32, device=dev)
        srcs = ptr_array([bufs[v % per].ptrs[v // per] if world > 1 else bufs[v % per].typed(torch.float32).data_ptr() for v in range(V)])

        def fused():
            check(lib.otb_grad_reduce(srcs, I(S), I(R), P(cs), P(cl), I(own), P(out), P(sos), stream_ptr()), "grad_reduce")

        def nccl_path():
            # one all_to_all per hosted bucket, then local ascending adds (order across ranks pinned by the rank index)
            acc = None
            for b in bufs:
                t = b.typed(torch.float32)
                recv = torch.empty_like(t)
                dist.all_to_all_single(recv, t)
                part = recv.view(world, -1)
                s = part[0].clone()
                for r in range(1, world):
                    s += part[r]
                acc = s if acc is None else acc.add_(s)
            acc.mul_(1.0 / V)
            return acc

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(a.iters):
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t.item()))
            return min(ts)

        ms = timed(fused)
        ms_nccl = timed(nccl_path) if world > 1 else None
        remote_bytes = 4.0 * (n / world) * (V - per)          # what one rank pulls from the other GPUs
        row = {"size_mb": 4.0 * n / (1 << 20), "S": S, "R": R, "gpus": world, "fused_ms": ms, "fused_busbw_GBs": remote_bytes / ms / 1e6,
               "frac_of_nvlink_peer_copy": remote_bytes / ms / 1e6 / NVLINK_PEER_GBS if world > 1 else None,
               "local_read_GBs": 4.0 * (n / world) * V / ms / 1e6, "nccl_a2a_ms": ms_nccl}
        if mb <= a.verify_mb:
            # every rank checks ITS slice of the result against the CPU fold of the same slice of all V buckets; the buckets
            # are seed-generated, so a rank regenerates each of them on its own GPU (one at a time) instead of gathering them
            fused()
            torch.cuda.synchronize()
            lo, hi = rank * own * CHUNK, (rank + 1) * own * CHUNK
            host = []
            for v in range(V):
                g = torch.Generator(device=dev).manual_seed(1234 + v)
                full = torch.randn(n, device=dev, generator=g) * 1e-3
                host.append(full[lo:hi].cpu())
                del full
            m = hi - lo
            ref = torch.zeros(m, dtype=torch.float32)
            rsos = torch.zeros(own, dtype=torch.float32)
            hcs = torch.arange(own, dtype=torch.int64) * CHUNK
            hcl = torch.full((own,), CHUNK, dtype=torch.int32)
            check(cpu_lib().otb_cpu_grad_reduce(ptr_array([t.data_ptr() for t in host]), I(S), I(R), P(hcs), P(hcl), I(own), P(ref), P(rsos)), "cpu")
            ok = torch.equal(out[lo:hi].cpu(), ref) and torch.equal(sos.cpu(), rsos)
            t = torch.tensor([1 if ok else 0], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
            row["bit_equal_to_cpu_fold"] = bool(t.item())
            del host, ref
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        for b in bufs:
            b.close()
        del bufs, out
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
