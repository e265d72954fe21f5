"""Several GPUs must reproduce the single-GPU bytes: same virtual topology, different process counts. The
gradient reduction and the weight redistribution run over CUDA-IPC peer pointers in this test."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.distributed]
WORKER = str(Path(__file__).resolve().parent / "multi_gpu_worker.py")


def _run(n, out, shard=4, **extra):
    env = dict(os.environ, OTB_TEST_OUT=str(out), OTB_TEST_SHARD=str(shard), NCCL_NVLS_ENABLE="0", **extra)
    if n == 1:
        cmd = [sys.executable, WORKER]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % n, "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), WORKER]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.load(open(out))


@pytest.mark.parametrize("shard", [4, 2])
def test_hashes_do_not_depend_on_the_gpu_count(tmp_path, shard):
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs at least 2 GPUs")
    one = _run(1, tmp_path / "g1.json", shard)
    assert one["status"] == 0
    for n in (2, 4):
        if n > n_gpus:
            break
        many = _run(n, tmp_path / ("g%d.json" % n), shard)
        assert many["status"] == 0
        assert many["hashes"] == one["hashes"], (n, many, one)
        # the reduction ran bucket by bucket under the last backward pass: in every step, or in every step after the first
        # where a process hosts one virtual rank (its first backward pass tells which parameters never get a gradient)
        assert many["overlapped_steps"] in (2, 3)


def test_message_transport_between_two_gpus_reproduces_the_single_gpu_hashes(tmp_path):
    """OTB_GRAD_TRANSPORT=collective on GPUs of one machine (NCCL point-to-point in place of peer loads): the transport of
    runs that span machines, checked against the single-GPU bytes"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    worker = str(Path(__file__).resolve().parent / "multi_gpu_worker.py")

    def run(n, out, **extra):
        env = dict(os.environ, OTB_TEST_OUT=str(out), OTB_TEST_SHARD="4", NCCL_NVLS_ENABLE="0", **extra)
        cmd = [sys.executable, worker] if n == 1 else [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % n,
                                                       "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        return json.load(open(out))

    one = run(1, tmp_path / "g1.json")
    two = run(2, tmp_path / "g2.json", OTB_GRAD_TRANSPORT="collective")
    assert one["status"] == 0 and two["status"] == 0 and two["hashes"] == one["hashes"]


def test_sharded_optimizer_state_over_peer_memory_reproduces_the_single_gpu_hashes(tmp_path):
    """OTB_STATE_SHARDING=1: each GPU allocates the moments and the reduced gradient of its own segments only; the reduction
    (bucket by bucket under the backward pass) and the AdamW kernel write through the packed offsets, and the bytes are those
    of one GPU that holds everything"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    one = _run(1, tmp_path / "g1.json")
    two = _run(2, tmp_path / "g2.json", OTB_STATE_SHARDING="1")
    assert one["status"] == 0 and two["status"] == 0 and two["packed_state"] and not one["packed_state"]
    assert two["hashes"] == one["hashes"]
    assert two["resident"]["moments"] < 0.6 * one["resident"]["moments"] and two["resident"]["reduced_gradient"] < 0.6 * one["resident"]["reduced_gradient"]
