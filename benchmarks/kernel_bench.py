"""Micro-benchmarks of the hot kernels on one B200, timed with CUDA events (warm-up, then best and median of N
runs; operands larger than L2 or an L2 flush between runs), with the library kernels of the same shape beside them
(cuBLAS through torch.matmul, flash-attn 2 when importable) and the achieved fraction of the measured peaks in
MEASURED_PEAKS.json.

  python benchmarks/kernel_bench.py gemm --shape qkv_fwd            # one named OPEN-1B GEMM
  python benchmarks/kernel_bench.py gemm --all
  python benchmarks/kernel_bench.py attn --window 0|512 [--bwd]
  python benchmarks/kernel_bench.py elementwise
Add --once to run the kernel a few times without timing (for profiler captures of a small case).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from open_transformers_b200.ops import functional as K

# (M, N, K, a_mn, b_mn, epi) at the OPEN-1B micro-batch (16384 tokens)
GEMMS = {
    "qkv_fwd": (16384, 3072, 2048, 0, 0, 0), "wo_fwd": (16384, 2048, 2048, 0, 0, 3), "gateup_fwd": (16384, 11264, 2048, 0, 0, 0),
    "down_fwd": (16384, 2048, 5632, 0, 0, 3), "lmhead_fwd": (16384, 128256, 2048, 0, 0, 0),
    "qkv_dgrad": (16384, 2048, 3072, 0, 1, 0), "gateup_dgrad": (16384, 2048, 11264, 0, 1, 0), "down_dgrad": (16384, 5632, 2048, 0, 1, 0),
    "lmhead_dgrad": (16384, 2048, 128256, 0, 1, 0),
    "qkv_wgrad": (3072, 2048, 16384, 1, 1, 2), "gateup_wgrad": (11264, 2048, 16384, 1, 1, 2), "down_wgrad": (2048, 5632, 16384, 1, 1, 2),
    "lmhead_wgrad": (128256, 2048, 16384, 1, 1, 2),
}


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def timeit(fn, iters=10, warm=3, flush=True):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return min(ts), statistics.median(ts)


def gemm_case(name, once=False):
    M, N, Kd, a_mn, b_mn, epi = GEMMS[name]
    A = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda").bfloat16()
    B = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda").bfloat16()
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if epi in (0, 3) else torch.float32)
    R = torch.randn(M, N, device="cuda").bfloat16() if epi == 3 else None

    def ours():
        K.gemm(A, B, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, epi=epi, residual=R)

    if once:
        for _ in range(3):
            ours()
        torch.cuda.synchronize()
        return {"name": name}
    At, Bt = (A.t() if a_mn else A), (B.t() if b_mn else B)
    best, med = timeit(ours)
    lbest, lmed = timeit(lambda: torch.matmul(At, Bt.t()))
    flops = 2.0 * M * N * Kd
    _, pk, how = peaks()
    return {"name": name, "M": M, "N": N, "K": Kd, "ms_best": best, "ms_median": med, "tflops": flops / best / 1e9,
            "frac_of_%s_cublas_peak" % how: flops / best / 1e9 / pk, "cublas_ms_best": lbest, "cublas_tflops": flops / lbest / 1e9}


def attn_case(window, bwd, once=False, B=4, T=4096, H=16, Hkv=4, D=128):
    qk = torch.randn(B * T, (H + Hkv) * D, device="cuda").bfloat16()
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, device="cuda").bfloat16()
    dO = torch.randn(B * T, H * D, device="cuda").bfloat16()
    O, lse = K.attn_fwd(qk, qkv, B, T, H, Hkv, D, window)
    dqk, dqkv = torch.empty_like(qk), torch.empty_like(qkv)
    fn = (lambda: K.attn_bwd(qk, qkv, O, dO, lse, dqk, dqkv, B, T, H, Hkv, D, window)) if bwd else (lambda: K.attn_fwd(qk, qkv, B, T, H, Hkv, D, window))
    if once:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        return {}
    best, med = timeit(fn, iters=8)
    pairs = sum(min(t + 1, window) for t in range(T)) if window else T * (T + 1) // 2
    flops = 4.0 * B * H * pairs * D * (2.5 if bwd else 1.0)
    res = {"window": window, "bwd": bwd, "ms_best": best, "ms_median": med, "tflops": flops / best / 1e9}
    try:
        from flash_attn import flash_attn_func
        q = torch.randn(B, T, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(B, T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn_like(k, requires_grad=True)
        ws = (-1, -1) if window == 0 else (window - 1, 0)
        if bwd:
            o = flash_attn_func(q, k, v, causal=True, window_size=ws)
            g = torch.randn_like(o)
            lb, _ = timeit(lambda: o.backward(g, retain_graph=True), iters=8)
        else:
            lb, _ = timeit(lambda: flash_attn_func(q, k, v, causal=True, window_size=ws), iters=8)
        res["flash_attn2_ms_best"] = lb
    except Exception as e:
        res["flash_attn2"] = "unavailable: %r" % e
    return res


def elementwise_cases():
    hbm, _, how = peaks()
    rows, D, F = 16384, 2048, 5632
    x = torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    gu = torch.randn(rows, 2 * F, device="cuda").bfloat16()
    dh = torch.randn(rows, F, device="cuda").bfloat16()
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    logits = torch.randn(rows, 128256, device="cuda").bfloat16()
    labels = torch.randint(0, 128256, (rows,), device="cuda")
    out = []
    for name, fn, nbytes in [
        ("rmsnorm_fwd", lambda: K.rmsnorm_fwd(x, w, 1e-5), 2 * rows * D * 2),
        ("rmsnorm_bwd", lambda: K.rmsnorm_bwd(y, x, w, rstd, True), 3 * rows * D * 2),
        ("swiglu_fwd", lambda: K.swiglu_fwd(gu), 3 * rows * F * 2),
        ("swiglu_bwd", lambda: K.swiglu_bwd(gu, dh), 5 * rows * F * 2),
        ("ce_zloss_fwd_bwd", lambda: K.ce_zloss_(logits, labels, 1e-4, 1.0 / rows, True), 2 * rows * 128256 * 2),
    ]:
        best, med = timeit(fn, iters=6)
        out.append({"name": name, "ms_best": best, "algorithmic_GBs": nbytes / best / 1e6, "frac_of_%s_hbm" % how: nbytes / best / 1e6 / hbm})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "elementwise"])
    ap.add_argument("--shape", default="qkv_fwd")
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    if a.what == "gemm":
        for n in (GEMMS if a.all else [a.shape]):
            print(json.dumps(gemm_case(n, a.once)), flush=True)
    elif a.what == "attn":
        print(json.dumps(attn_case(a.window, a.bwd, a.once)))
    else:
        for r in elementwise_cases():
            print(json.dumps(r), flush=True)
    print(json.dumps({"kernel_status": K.kernel_status("cuda")}))


if __name__ == "__main__":
    main()
