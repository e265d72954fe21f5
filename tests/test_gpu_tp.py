"""Tensor-parallel GEMM kernels. On one GPU the chained GEMM is run rank by rank (each rank's launch completes before
the next starts, so nothing waits on a concurrent kernel) and must reproduce the unsplit GEMM bit for bit, which
exercises the accumulator hand-over through tensor memory; with two or more GPUs the real peer-memory path runs
under torchrun, all-gather -> GEMM included."""
import ctypes
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import free_port
from open_transformers_b200.ops import functional as K
from open_transformers_b200.ops.functional import _status
from open_transformers_b200.ops.native import I, L, P as PTR, check, cuda_lib, stream_ptr
from open_transformers_b200.parallel.tensor_parallel import TpWorkspace, _ptrs

pytestmark = pytest.mark.gpu
WORKER = str(Path(__file__).resolve().parent / "tp_worker.py")


@pytest.mark.parametrize("P,M,N,Kd,b_mn", [(2, 512, 512, 1024, False), (4, 1024, 384, 2048, False), (4, 512, 2048, 5632, True)])
def test_chained_gemm_rank_by_rank_equals_unsplit(P, M, N, Kd, b_mn):
    dev = torch.device("cuda")
    lib = cuda_lib()
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
    w = (torch.randn(N, Kd, generator=g) * 0.05).bfloat16().to(dev)
    r = torch.randn(M, N, generator=g).bfloat16().to(dev)
    bn = lib.otb_tp_chain_bn(I(N))
    tiles = (M // 128) * ((N + bn - 1) // bn)
    inbox = [torch.zeros(M, N, device=dev) for _ in range(P)]
    result = [torch.zeros(M, N, device=dev) for _ in range(P)]
    fl_in = [torch.zeros(tiles * 4, dtype=torch.int32, device=dev) for _ in range(P)]
    fl_res = [torch.zeros(tiles * 4, dtype=torch.int32, device=dev) for _ in range(P)]
    st = PTR(_status(dev))
    for seq in (1, 2):
        for rank in range(P):
            ks = slice(rank * (Kd // P), (rank + 1) * (Kd // P))
            a = x[:, ks].contiguous()
            b = w[:, ks].t().contiguous() if b_mn else w[:, ks].contiguous()
            if rank == P - 1:
                outs, oflags = [t.data_ptr() for t in result], [t.data_ptr() for t in fl_res]
            else:
                outs, oflags = [inbox[rank + 1].data_ptr()], [fl_in[rank + 1].data_ptr()]
            check(lib.otb_tp_chain_gemm(PTR(a), PTR(b), I(M), I(N), I(Kd // P), L(a.stride(0)), L(b.stride(0)), I(b_mn), PTR(inbox[rank]),
                                        PTR(fl_in[rank]), _ptrs(outs), _ptrs(oflags), L(N), I(rank), I(P), ctypes.c_uint(seq), st, stream_ptr()),
                  "tp_chain_gemm")
            torch.cuda.synchronize()
        want = K.gemm(x, w, epi=K.EPI_RESIDUAL, residual=r)
        for rank in range(P):
            rows = slice(rank * (M // P), (rank + 1) * (M // P))
            y = torch.empty(M // P, N, dtype=torch.bfloat16, device=dev)
            rs = r[rows].contiguous()
            check(lib.otb_tp_finish(PTR(result[rank]), PTR(fl_res[rank]), ctypes.c_uint(seq), PTR(rs), PTR(y), I(M), I(N), I(rank), I(P), L(N),
                                    L(rs.stride(0)), L(y.stride(0)), st, stream_ptr()), "tp_finish")
            assert torch.equal(y, want[rows]), "rank %d rows differ in %d elements" % (rank, int((y != want[rows]).sum()))
    assert K.kernel_status(dev) == 0


def test_single_rank_workspace_is_the_plain_gemm():
    dev = torch.device("cuda")
    ws = TpWorkspace(dev, 0, 1)
    g = torch.Generator().manual_seed(8)
    x = torch.randn(256, 512, generator=g).bfloat16().to(dev)
    w = torch.randn(384, 512, generator=g).bfloat16().to(dev)
    c, xf = ws.ag_gemm("a", x, w)
    assert torch.equal(c, K.gemm(x, w)) and torch.equal(xf, x)
    assert torch.equal(ws.chain_gemm("c", x, w), K.gemm(x, w))
    ws.barrier()
    torch.cuda.synchronize()
    assert K.kernel_status(dev) == 0
    ws.close()


@pytest.mark.distributed
def test_peer_memory_kernels_equal_the_unsplit_gemm(tmp_path):
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs at least 2 GPUs")
    for n in (2, 4):
        if n > n_gpus:
            break
        out = tmp_path / ("tp%d.json" % n)
        env = dict(os.environ, OTB_TEST_OUT=str(out), NCCL_NVLS_ENABLE="0")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % n, "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), WORKER]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        for rank, res in enumerate(json.load(open(out))):
            assert res.pop("status") == 0, (n, rank)
            assert all(all(v) for v in res.values()), (n, rank, res)
