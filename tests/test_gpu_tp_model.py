"""Tensor-parallel MODEL step on GPUs: a group of 2 GPUs must write the hashes, losses and gradient norms of the single-GPU
run of the same bf16 model, with NCCL all-gathers around the tcgen05 kernels and with the fused peer-memory kernels
(`run.tp_fused`); two groups of two on four GPUs likewise."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.distributed]
WORKER = str(Path(__file__).resolve().parent / "tp_cpu_worker.py")


def _run(n, tp, out, extra=""):
    env = dict(os.environ, OTB_TEST_OUT=str(out), OTB_TEST_TP=str(tp), OTB_TEST_BF16="1", OTB_TEST_DEVICE="cuda", OTB_TEST_T="128", NCCL_NVLS_ENABLE="0",
               OTB_TEST_EXTRA=extra)
    if n == 1:
        cmd = [sys.executable, WORKER]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % n, "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), WORKER]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.load(open(out))


def test_tensor_parallel_pair_of_gpus_reproduces_the_single_gpu_bytes(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    one = _run(1, 1, tmp_path / "g1.json")
    two = _run(2, 2, tmp_path / "g2.json")
    assert two == one, (two, one)


def test_two_tensor_parallel_groups_on_four_gpus_reproduce_the_single_gpu_hashes(tmp_path):
    """TP = 2 x DP = 2: each group hosts one virtual rank; gradient buffers cross by NCCL all-gather"""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least 4 GPUs")
    one = _run(1, 1, tmp_path / "g1.json")
    four = _run(4, 2, tmp_path / "g4.json")
    assert [h for _, _, h in four] == [h for _, _, h in one]
    assert [n for n, _, _ in four] == [n for n, _, _ in one]


def test_fused_peer_memory_kernels_carry_the_tensor_parallel_model_step(tmp_path):
    """run.tp_fused: all-gather -> GEMM and chained GEMM -> ordered reduction inside the model step; same bytes as one GPU"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    one = _run(1, 1, tmp_path / "g1.json")
    two = _run(2, 2, tmp_path / "g2.json", "run.tp_fused=true")
    assert two == one, (two, one)
