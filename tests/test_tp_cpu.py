"""Tensor parallelism on CPU ranks: a tensor-parallel group of 2 gloo processes (and 2 groups of 2) must write the very
hashes, losses and gradient norms of the single-process run - fp32 (exact family) and bf16 (tensor-core model twin)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from helpers import free_port

WORKER = str(Path(__file__).resolve().parent / "tp_cpu_worker.py")


_single: dict = {}


def _run(world, tp, bf16, out, extra="", **env_extra):
    if world == 1:  # several tests compare with the same single-process run: compute each once
        key = (bf16, extra, tuple(sorted(env_extra.items())))
        if key not in _single:
            _single[key] = _launch(world, tp, bf16, out, extra, **env_extra)
        return _single[key]
    return _launch(world, tp, bf16, out, extra, **env_extra)


def _launch(world, tp, bf16, out, extra="", **env_extra):
    port = free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2", OTB_TEST_TP=str(tp), OTB_TEST_BF16="1" if bf16 else "0", OTB_TEST_OUT=str(out), OTB_TEST_EXTRA=extra, **env_extra)
        procs.append(subprocess.Popen([sys.executable, WORKER], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(o.decode())
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)[-6000:]
    return json.load(open(out))


@pytest.mark.distributed
@pytest.mark.parametrize("bf16", [False, True])
def test_tensor_parallel_group_reproduces_the_single_process_bytes(tmp_path, bf16):
    base = _run(1, 1, bf16, tmp_path / "base.json")
    tp2 = _run(2, 2, bf16, tmp_path / "tp2.json")
    assert tp2 == base, (tp2, base)


@pytest.mark.distributed
def test_two_tensor_parallel_groups_share_the_virtual_ranks(tmp_path):
    base = _run(1, 1, False, tmp_path / "base.json")
    got = _run(4, 2, False, tmp_path / "tp2dp2.json")          # TP = 2 x DP = 2: each group hosts one virtual rank
    assert [h for _, _, h in got] == [h for _, _, h in base]
    assert [n for n, _, _ in got] == [n for n, _, _ in base]


@pytest.mark.distributed
def test_qk_norm_gains_under_tensor_parallelism(tmp_path):
    """heads are split over the group, the gains' gradients run over all (token, head) rows in the unsplit order"""
    extra = "model.modules.attention=gqa_qknorm_repop model.qk_norm=true model.qk_norm_gain=true model.n_heads=4 model.n_kv_heads=2 model.head_dim=32"
    base = _run(1, 1, False, tmp_path / "base.json", extra)
    tp2 = _run(2, 2, False, tmp_path / "tp2.json", extra)
    assert tp2 == base, (tp2, base)
    plain = _run(1, 1, False, tmp_path / "plain.json", extra.replace("qk_norm_gain=true", "qk_norm_gain=false"))
    assert plain[-1][2] != base[-1][2]


@pytest.mark.distributed
def test_activation_checkpointing_under_tensor_parallelism(tmp_path):
    """the recomputed forward repeats the group's gathers in the same order on every rank; no bit changes"""
    base = _run(1, 1, False, tmp_path / "base.json")
    tp2 = _run(2, 2, False, tmp_path / "tp2.json", "run.activation_checkpoint=true")
    assert tp2 == base, (tp2, base)


@pytest.mark.distributed
def test_fused_kernel_call_sites_of_the_model_step(tmp_path):
    """the model step routed through the workspace's two fused operations (a host stand-in with their documented meaning):
    operand layouts, keys and saved tensors of the three call sites give the unsplit bytes"""
    base = _run(1, 1, True, tmp_path / "base.json", OTB_TEST_T="128")
    tp2 = _run(2, 2, True, tmp_path / "tp2.json", OTB_TEST_T="128", OTB_TEST_HOST_WS="1")
    assert tp2 == base, (tp2, base)


@pytest.mark.distributed
@pytest.mark.parametrize("method", ["lsq", "absmax"])
def test_quantisation_aware_layers_under_tensor_parallelism(tmp_path, method):
    """W8A8 layers split over the group: whole-activation absmax, exact integer products, unsplit float reductions"""
    extra = "++model.qat.enabled=true ++model.qat.method=%s ++model.qat.scale_refresh_every_n_steps=2" % method
    bf16 = method == "lsq"  # one method on the tensor-core twin, the other on the exact fp32 family
    base = _run(1, 1, bf16, tmp_path / "base.json", extra)
    tp2 = _run(2, 2, bf16, tmp_path / "tp2.json", extra)
    assert tp2 == base, (tp2, base)
    plain = _run(1, 1, bf16, tmp_path / "plain.json")
    assert plain[-1][2] != base[-1][2]


@pytest.mark.distributed
def test_ddp_mode_uses_the_library_all_reduce_and_is_refused_by_the_audit(tmp_path):
    """run.parallel=ddp: gradients summed by the backend's all-reduce (order not pinned, so only closeness is asked)"""
    from open_transformers_b200.cli.audit_replay import AuditError, audit_replay

    base = _run(1, 1, False, tmp_path / "base.json")
    ddp = _run(2, 1, False, tmp_path / "ddp.json", "run.parallel=ddp")
    for (n0, _, _), (n1, _, _) in zip(base, ddp):
        assert abs(n1 - n0) <= 1e-5 * n0
    with pytest.raises(AuditError):
        audit_replay(from_init=True, config_name="tiny_cpu", overrides=["run.parallel=ddp", "run.virtual_dp_size=2"], until_step=1)


@pytest.mark.distributed
@pytest.mark.parametrize("world,bf16", [(2, True), (4, False)])
def test_sharded_ownership_over_point_to_point_messages(tmp_path, world, bf16):
    """OTB_GRAD_TRANSPORT=collective (what GPUs on several machines use): every process sends each owner its segments, the
    owner reduces, updates and digests them, new weights come back by all-gather; four virtual ranks on 2 or 4 processes
    write the single-process hashes, losses and norms"""
    env = dict(OTB_TEST_V="4", OTB_TEST_TD="tree")
    base = _run(1, 1, bf16, tmp_path / "base.json", **env)
    got = _run(world, 1, bf16, tmp_path / "sharded.json", OTB_GRAD_TRANSPORT="collective", **env)
    assert [h for _, _, h in got] == [h for _, _, h in base]
    assert [n for n, _, _ in got] == [n for n, _, _ in base]


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_optimizer_state_keeps_only_owned_segments_and_writes_the_same_hashes(tmp_path, world):
    """run.state_sharding / OTB_STATE_SHARDING=1: the AdamW moments and the reduced gradient are allocated for the segments a
    process owns only (about 1/N of the full layout each); reductions, updates, digests, gathered state and resident-byte
    accounting agree with the single-process run"""
    import torch

    env = dict(OTB_TEST_V="4", OTB_TEST_TD="tree")
    base = _run(1, 1, True, tmp_path / "base.json", OTB_TEST_STATE_OUT=str(tmp_path / "base.pt"), **env)
    got = _run(world, 1, True, tmp_path / "packed.json", OTB_GRAD_TRANSPORT="collective", OTB_STATE_SHARDING="1",
               OTB_TEST_STATE_OUT=str(tmp_path / "packed.pt"), **env)
    assert [(n, h) for n, _, h in got] == [(n, h) for n, _, h in base]
    a, b = torch.load(tmp_path / "base.pt"), torch.load(tmp_path / "packed.pt")
    for kind in ("m1", "m2", "grad"):
        for name, t in a[kind].items():
            assert torch.equal(t, b[kind][name]), (kind, name)
    full, part = a["resident"], b["resident"]
    assert part["master"] == full["master"]
    for key in ("moments", "reduced_gradient"):
        assert part[key] < full[key] * (1.0 / world + 0.2), (key, part[key], full[key])
