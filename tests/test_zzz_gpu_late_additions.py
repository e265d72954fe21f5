"""GPU tests of paths that are Python around already verified kernels and were added after the last run on a GPU; they sort
last so that a surprise here cannot hide the results of the established tests: the Hadamard int8 product against its CPU
twin, optimizer moments leaving the GPU between steps, the model step on the fused peer-memory kernels (2 GPUs) and two
tensor-parallel groups over NCCL gathers (4 GPUs)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import free_port
from open_transformers_b200.config import load_config
from open_transformers_b200.ops import functional as K
from open_transformers_b200.train.engine import TrainEngine
from test_gpu_engine import _run as _engine_run

pytestmark = pytest.mark.gpu
WORKER = str(Path(__file__).resolve().parent / "tp_cpu_worker.py")


def _both(fn, *cpu_args):
    return fn(*cpu_args), fn(*[t.cuda() if isinstance(t, torch.Tensor) else t for t in cpu_args])


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


def test_gpu_hadamard_int8_product_bitwise_vs_cpu():
    """rotation (IEEE adds), row statistics, quantiser and the tcgen05 kind::i8 GEMM give the CPU twin's bits"""
    g = torch.Generator().manual_seed(8)
    a, b = torch.randn(256, 384, generator=g), torch.randn(136, 384, generator=g).bfloat16()
    a[5, 100] = 90.0
    cpu, gpu = _both(lambda a_, b_: K.ste_matmul_hadamard(a_, b_), a, b)
    assert torch.equal(cpu, gpu.cpu()), "%d elements differ" % int((cpu != gpu.cpu()).sum())
    assert K.kernel_status("cuda") == 0


def test_offloaded_moments_leave_the_gpu_between_steps_and_change_no_bit(tmp_path):
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.vocab_size=4096", "train.seq_len=256", "data.seq_len=256",
                                      "run.virtual_dp_size=2", "run.dp_shard_size=2"])
    want = [h for _, _, h in _engine_run(cfg, "cuda", steps=3, T=256, vocab=4096, td="tree")]
    eng = TrainEngine(cfg, "cuda", offload_optimizer=True, optimizer_offload_dir=str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prev, got = None, []
    for _ in range(3):
        eng.zero_grads()
        for v in range(2):
            ids = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            lab = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            eng.forward_backward(v, ids, lab, 1)
        assert got == [] or eng._m1 is None  # absent during forward and backward
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        prev = eng.sharded_state_hash(prev, None, tensor_digest="tree")
        got.append(prev)
        eng.release_state()
    assert got == want
    eng.close()


@pytest.mark.distributed
def test_two_tensor_parallel_groups_on_four_gpus_reproduce_the_single_gpu_hashes(tmp_path):
    """TP = 2 x DP = 2: each group hosts one virtual rank; gradient buffers cross by NCCL all-gather"""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least 4 GPUs")
    one = _run(1, 1, tmp_path / "g1.json")
    four = _run(4, 2, tmp_path / "g4.json")
    assert [h for _, _, h in four] == [h for _, _, h in one]
    assert [n for n, _, _ in four] == [n for n, _, _ in one]


@pytest.mark.distributed
def test_fused_peer_memory_kernels_carry_the_tensor_parallel_model_step(tmp_path):
    """run.tp_fused: all-gather -> GEMM and chained GEMM -> ordered reduction inside the model step; same bytes as one GPU"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    one = _run(1, 1, tmp_path / "g1.json")
    two = _run(2, 2, tmp_path / "g2.json", "run.tp_fused=true")
    assert two == one, (two, one)


@pytest.mark.distributed
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
