"""Tensor-parallel GEMM micro-benchmark at the OPEN-1B layer shapes (one node, P GPUs, torch.distributed.run).

Two fused kernels against their library baselines, every number timed on the device with CUDA events around a loop of
``--iters`` calls and reduced to the max over ranks:

* all-gather -> GEMM (QKV and gate/up projections): ``TpWorkspace.ag_gemm`` (one kernel; peer stores + tcgen05) vs
  NCCL ``all_gather_into_tensor`` followed by a cuBLAS matmul;
* GEMM -> ordered reduction (attention output and down projections): ``TpWorkspace.chain_gemm`` (accumulator tiles
  travel rank to rank inside the tensor-core accumulation; bit-identical to the unsplit GEMM) vs a cuBLAS matmul
  followed by NCCL ``reduce_scatter_tensor`` of bf16 partial sums (which is NOT bit-identical to the unsplit GEMM).

Roofline per call = the slower of (FLOPs of one rank / measured bf16 peak) and (bytes that must cross one NVLink
direction of one GPU / 770 GB/s, the measured peer-copy bandwidth); ``frac`` = roofline / achieved time.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29541 \
      benchmarks/tp_gemm_bench.py --tokens 16384
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
from open_transformers_b200.parallel.tensor_parallel import TpWorkspace

NVLINK_PEER_GBS = 770.0


def peak_tflops() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops"])
    except Exception:
        return 1590.0


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
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=5632)
    ap.add_argument("--qkv", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--copier-ctas", type=int, default=16)
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    P, M, d = world, a.tokens, a.d_model
    ws = TpWorkspace(dev, rank, P, None, copier_ctas=a.copier_ctas)
    peak = peak_tflops() * 1e12
    g = torch.Generator().manual_seed(rank)
    rows = ws.shard_rows(M)
    out = []

    # ---- all-gather -> GEMM
    for name, N in (("qkv", a.qkv), ("gate_up", 2 * a.ffn)):
        Np = N // P
        x_shard = ws.site(name, M, d).full[rows]  # the producing kernel writes its rows straight into the gathered buffer
        x_shard.copy_(torch.randn(M // P, d, generator=g).bfloat16())
        w = (torch.randn(Np, d, generator=g) * 0.02).bfloat16().to(dev)
        x_full = torch.empty(M, d, dtype=torch.bfloat16, device=dev)

        def fused():
            ws.barrier()
            ws.ag_gemm(name, x_shard, w)

        def library():
            if P > 1:
                dist.all_gather_into_tensor(x_full, x_shard)
            else:
                x_full.copy_(x_shard)
            torch.matmul(x_full, w.t())

        t_f, t_l = timed(fused, a.iters, world), timed(library, a.iters, world)
        flops = 2.0 * M * Np * d
        nv_bytes = (P - 1) / P * M * d * 2
        roof = max(flops / peak, nv_bytes / (NVLINK_PEER_GBS * 1e9)) * 1e3
        out.append({"op": "all_gather->gemm " + name, "P": P, "M": M, "N_per_rank": Np, "K": d, "fused_ms": t_f, "nccl_cublas_ms": t_l,
                    "roofline_ms": roof, "frac_of_roofline": roof / t_f, "tflops_per_gpu": flops / t_f / 1e9})

    # ---- GEMM -> ordered reduction over ranks
    for name, Kfull in (("attn_out", d), ("ffn_down", a.ffn)):
        Kr = Kfull // P
        x = torch.randn(M, Kr, generator=g).bfloat16().to(dev)
        w = (torch.randn(d, Kr, generator=g) * 0.02).bfloat16().to(dev)
        res = torch.randn(M // P, d, generator=g).bfloat16().to(dev)
        y_shard = torch.empty(M // P, d, dtype=torch.bfloat16, device=dev)

        def fused():
            ws.barrier()
            ws.chain_gemm(name, x, w, residual_shard=res)

        def library():
            part = torch.matmul(x, w.t())
            if P > 1:
                dist.reduce_scatter_tensor(y_shard, part)
            else:
                y_shard.copy_(part)
            y_shard.add_(res)

        t_f, t_l = timed(fused, a.iters, world), timed(library, a.iters, world)
        flops = 2.0 * M * d * Kr
        nv_bytes = M * d * 4.0 if P > 1 else 0.0   # one fp32 accumulator hand-over per link direction
        roof = max(flops / peak, nv_bytes / (NVLINK_PEER_GBS * 1e9)) * 1e3
        out.append({"op": "gemm->ordered_reduce " + name, "P": P, "M": M, "N": d, "K_per_rank": Kr, "fused_ms": t_f, "nccl_cublas_ms": t_l,
                    "roofline_ms": roof, "frac_of_roofline": roof / t_f, "tflops_per_gpu": flops / t_f / 1e9,
                    "note": "library path sums bf16 partials in NCCL order: not bit-identical to the unsplit GEMM"})
    torch.cuda.synchronize()
    status = K.kernel_status(dev)
    if rank == 0:
        for row in out:
            row["kernel_status"] = status
            print(json.dumps(row))
    if world > 1:
        dist.barrier()
    ws.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
