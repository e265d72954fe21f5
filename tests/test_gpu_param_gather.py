"""Parameter all-gather fused into the consuming GEMM (`otb_pg_gemm`, `parallel/param_gather.py`).

The kernel pulls rows through pointers and waits only for copier warps of its own launch, so the processes of a run can
be stood in for by buffers of ONE GPU: "process p" is a full-size buffer in which only p's rows are valid and everything
else is poisoned. The engine-level test needs two GPUs."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import free_port

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _buffers(W, P, seg_begin, rpo):
    """Per process a poisoned copy of W with only its own rows valid."""
    N = W.shape[0]
    ends = seg_begin[1:] + [N]
    bufs = []
    for p in range(P):
        b = torch.full_like(W, float("nan"))
        for b0, e0, r in zip(seg_begin, ends, rpo):
            lo = min(b0 + p * r, e0)
            hi = e0 if p == P - 1 else min(b0 + (p + 1) * r, e0)
            b[lo:hi] = W[lo:hi]
        bufs.append(b)
    return bufs


@pytest.mark.parametrize("P,M,seg_rows,K_", [(4, 1024, [1024], 512),            # one weight, 256 rows per owner
                                            (8, 640, [704, 704], 328 * 8 // 8),  # two weights, owners change inside a 128-row block
                                            (2, 384, [512, 128, 128], 256),      # wq|wk|wv: three weights in one operand
                                            (8, 256, [200], 64)])                # fewer rows than owners x 128, ragged edge
def test_gathering_gemm_equals_the_plain_gemm_and_completes_the_local_buffer(P, M, seg_rows, K_):
    from open_transformers_b200.ops import functional as K
    from open_transformers_b200.parallel.param_gather import GatheredWeight, flag_words

    g = torch.Generator().manual_seed(5)
    N = sum(seg_rows)
    W = torch.randn(N, K_, generator=g).bfloat16().to(DEV)
    x = torch.randn(M, K_, generator=g).bfloat16().to(DEV)
    res = torch.randn(M, N, generator=g).bfloat16().to(DEV)
    seg_begin = [sum(seg_rows[:j]) for j in range(len(seg_rows))]
    rpo = [-(-r // P) for r in seg_rows]
    want = K.gemm(x, W)
    want_res = K.gemm(x, W, epi=K.EPI_RESIDUAL, residual=res)
    want_f32 = K.gemm(x, W, epi=K.EPI_STORE_F32)
    for rank in sorted({0, P // 2, P - 1}):
        bufs = _buffers(W, P, seg_begin, rpo)
        flags = torch.zeros(flag_words(N), dtype=torch.int32, device=DEV)
        unit = 128 if N >= 16384 else (64 if N >= 8192 else 16)   # rows per copy unit, as the kernel cuts them
        gw = GatheredWeight(bufs[rank], [b.data_ptr() for b in bufs], rank, seg_begin, rpo, flags)
        gw.epoch = 1
        assert gw.pending()
        got = gw.gemm(x)
        torch.cuda.synchronize()
        assert K.kernel_status(torch.device(DEV)) == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), rank
        assert torch.equal(bufs[rank].view(torch.int16), W.view(torch.int16)), "the local buffer must hold the whole weight afterwards"
        assert not gw.pending() and int(flags[-1]) == -(-N // unit) and int(flags[:-1].sum()) == -(-N // unit)
        for p in range(P):                                          # nobody else's buffer was written
            if p != rank:
                assert torch.isnan(bufs[p].float()).any() or P == 1
        # the next update: new rows on the owners, a residual epilogue and an fp32 store this time
        gw.epoch = 2
        bufs2 = _buffers(W, P, seg_begin, rpo)
        for p in range(P):
            if p != rank:
                bufs[p].copy_(bufs2[p])
        assert torch.equal(gw.gemm(x, res).view(torch.int16), want_res.view(torch.int16))
        gw.epoch = 3
        assert torch.equal(gw.gemm(x, out_fp32=True), want_f32)
        assert int(flags[-1]) == 3 * -(-N // unit)                 # the counters only grow: three pulls so far
        assert K.kernel_status(torch.device(DEV)) == 0


WORKER = str(Path(__file__).resolve().parent / "multi_gpu_worker.py")


@pytest.mark.distributed
@pytest.mark.parametrize("sharded_state", [False, True])
def test_gather_mode_on_two_gpus_reproduces_the_replicated_hashes(tmp_path, sharded_state):
    """run.param_sharding=gather: the AdamW kernel keeps the projection weights' new rows on their owner and the first
    forward GEMM of the next step pulls them over peer memory; hashes are those of the default mode and of one GPU.
    ``sharded_state``: together with moments and reduced gradient allocated for the owned segments only"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")

    def run(n, out, **extra):
        env = dict(os.environ, OTB_TEST_OUT=str(out), OTB_TEST_SHARD="4", NCCL_NVLS_ENABLE="0", **extra)
        cmd = [sys.executable, WORKER] if n == 1 else [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % n,
                                                       "--master-addr", "127.0.0.1", "--master-port", str(free_port()), WORKER]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        return json.load(open(out))

    one = run(1, tmp_path / "g1.json")
    extra = {"OTB_STATE_SHARDING": "1"} if sharded_state else {}
    two = run(2, tmp_path / "g2.json", OTB_PARAM_SHARDING="gather", **extra)
    assert one["status"] == 0 and two["status"] == 0 and two["packed_state"] == sharded_state
    assert two["hashes"] == one["hashes"]
    assert two["gather_calls"] > 0 and one["gather_calls"] == 0
