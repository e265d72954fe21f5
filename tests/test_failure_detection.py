"""Failure detection. On the host with CPU (gloo) ranks: a rank that leaves between steps is noticed by the heartbeat
before the survivor's next collective; a rank that never joins ends the rendezvous with an error after the configured
timeout; SIGTERM produces an off-cadence checkpoint whose hash replays; run-id disagreement and a missing per-rank file
are loud. On one GPU (marked `gpu`): the bounded in-kernel waits on a peer's flag are given a few milliseconds and a flag
that nothing sets; each kernel must write its status word and return, leaving the context usable. Nothing here makes a
device fault, trap or hang."""
import json
import os
import subprocess
import sys
import textwrap
import time
from pathlib import Path

import pytest

from helpers import free_port, tiny_cfg

ROOT = Path(__file__).resolve().parent.parent


def _spawn(script_text, tmp, world, name, extra_env=None, ranks=None):
    script = Path(tmp) / (name + ".py")
    script.write_text(script_text)
    port, hb_port = free_port(), free_port()
    procs = []
    for rank in (ranks if ranks is not None else range(world)):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OTB_HEARTBEAT_PORT=str(hb_port), OMP_NUM_THREADS="2", **(extra_env or {}))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    return procs


def _finish(procs, timeout):
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out.decode())
    return outs


HEARTBEAT_WORKER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, {root!r})
    from open_transformers_b200.parallel.heartbeat import Heartbeat, PeerFailure
    rank, port = int(os.environ["RANK"]), int(os.environ["HB_PORT"])
    hb = Heartbeat(rank, 2, "127.0.0.1", port, interval_s=0.1, timeout_s=1.5)
    mode = os.environ["HB_MODE"]
    t0 = time.time()
    if rank == 1:
        time.sleep(0.5)
        if mode == "notice":
            hb.report_failure("ValueError: boom at step 3")       # leaves between steps and says so
            time.sleep(0.3)
        os._exit(3)                                               # mode "silent": just dies, no notice
    try:
        while time.time() - t0 < 20:
            hb.check()                                            # what the train loop does before every step
            time.sleep(0.05)
        print("NOT DETECTED")
        sys.exit(1)
    except PeerFailure as e:
        print("DETECTED rank=%d after %.2f s: %s" % (e.rank, time.time() - t0, e.reason))
        sys.exit(0)
""")


@pytest.mark.distributed
@pytest.mark.parametrize("mode", ["notice", "silent"])
def test_heartbeat_reports_a_rank_that_left(tmp_path, mode):
    port = free_port()
    procs = _spawn(HEARTBEAT_WORKER.format(root=str(ROOT)), tmp_path, 2, "hb_" + mode, {"HB_PORT": str(port), "HB_MODE": mode})
    outs = _finish(procs, 60)
    assert procs[0].returncode == 0, outs[0]
    assert "DETECTED rank=1" in outs[0]
    if mode == "notice":
        assert "boom at step 3" in outs[0]
    else:
        assert "no heartbeat" in outs[0]
    assert procs[1].returncode == 3


TRAIN_WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
    from helpers import tiny_cfg
    import open_transformers_b200.train.loop as loop
    from open_transformers_b200.parallel.heartbeat import PeerFailure
    rank = int(os.environ["RANK"])
    cfg = tiny_cfg({tmp!r}, ["run.run_id=hb", "run.heartbeat_timeout_s=2", "train.ckpt_every_steps=0"])
    if rank == 1:
        steps = {{"n": 0}}
        real = loop.TrainEngine.optimizer_step
        def failing(self, lr, clip):
            steps["n"] += 1
            if steps["n"] == 2:
                raise RuntimeError("injected host failure on rank 1")     # raised between kernels, on the host
            return real(self, lr, clip)
        loop.TrainEngine.optimizer_step = failing
    try:
        loop.train(cfg, device="cpu", data_root={tmp!r})
        print("FINISHED")
    except PeerFailure as e:
        print("PEER FAILURE SEEN BY %d: %s" % (rank, e))
        os._exit(7)
    except RuntimeError as e:
        print("RANK %d RAISED: %s" % (rank, e))
        os._exit(5)
""")


@pytest.mark.distributed
def test_survivor_of_a_failed_rank_stops_instead_of_hanging(tmp_path):
    tmp = str(tmp_path)
    tiny_cfg(tmp)  # synthetic shards written once, before the ranks start
    procs = _spawn(TRAIN_WORKER.format(root=str(ROOT), tmp=tmp), tmp, 2, "train_hb")
    t0 = time.time()
    outs = _finish(procs, 120)
    assert time.time() - t0 < 100
    assert procs[1].returncode == 5 and "injected host failure" in outs[1], outs[1]
    # rank 0 either learns of it from the notice at its next heartbeat check, or its collective errors because the peer is gone
    assert procs[0].returncode != 0, outs[0]
    assert "FINISHED" not in outs[0]


NEVER_JOINS = textwrap.dedent("""
    import sys, time
    sys.path.insert(0, {root!r})
    from open_transformers_b200.parallel.env import init_distributed
    t0 = time.time()
    try:
        init_distributed("cpu", timeout_s=3)
        print("JOINED")
    except Exception as e:
        print("RENDEZVOUS FAILED after %.1f s: %s" % (time.time() - t0, type(e).__name__))
        sys.exit(4)
""")


@pytest.mark.distributed
def test_a_rank_that_never_joins_ends_the_rendezvous_with_an_error(tmp_path):
    procs = _spawn(NEVER_JOINS.format(root=str(ROOT)), tmp_path, 2, "never", ranks=[0])   # rank 1 is never started
    outs = _finish(procs, 90)
    assert procs[0].returncode == 4, outs[0]
    assert "RENDEZVOUS FAILED" in outs[0]


def test_sigterm_checkpoint_is_off_cadence_and_replays(tmp_path, monkeypatch):
    """SIGTERM is polled after the optimizer step; the run checkpoints at that step, records the hash and exits 0."""
    import open_transformers_b200.train.loop as loop
    from open_transformers_b200.cli.audit_replay import audit_replay

    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=0", "run.run_id=term"])
    calls = {"n": 0}

    def fake(world, device, group=None):
        calls["n"] += 1
        return calls["n"] == 2          # "SIGTERM arrived" during the second step

    monkeypatch.setattr(loop, "_emergency_exit_requested", fake)
    with pytest.raises(SystemExit) as e:
        loop.train(cfg, device="cpu", data_root=tmp)
    assert e.value.code == 0
    run = Path(tmp) / "runs" / "term"
    ck = run / "checkpoints" / "step_000000002"
    assert (ck / "_COMPLETE").exists()
    logged = [json.loads(l) for l in (run / "logs" / "state_hashes.jsonl").read_text().splitlines()]
    at2 = [r["state_hash"] for r in logged if r.get("step") == 2]
    assert at2 and (ck / "state_hash.txt").read_text().strip() == at2[-1]
    r = audit_replay(None, from_init=True, descriptor_checkpoint=str(ck), until_step=2, data_root=tmp)
    assert r["match"] is True


def test_missing_per_rank_file_and_run_id_disagreement_are_loud(tmp_path):
    from open_transformers_b200.train.checkpoint import Checkpointer
    from open_transformers_b200.train.engine import TrainEngine
    from open_transformers_b200.train.loop import _assert_same_on_all_ranks, train

    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=2", "run.run_id=files"])
    train(cfg, device="cpu", data_root=tmp, max_steps=2)
    ck = Path(tmp) / "runs" / "files" / "checkpoints" / "step_000000002"
    (ck / "batch_hasher.rank_1.bin").unlink()
    eng = TrainEngine(cfg, "cpu", init=False)
    with pytest.raises(FileNotFoundError):
        Checkpointer(ck.parent.parent).load(str(ck), eng)
    eng.close()
    _assert_same_on_all_ranks("x", "run_id", 1)   # a single process trivially agrees with itself


@pytest.mark.distributed
@pytest.mark.parametrize("how", ["tcp_store", "file_store"])
def test_rendezvous_through_a_tcp_store_or_a_file_store(tmp_path, how):
    """DIST_MASTER_FQDN / DIST_MASTER_STORE_PORT and TORCH_DIST_STORE_FILE replace the env:// variables"""
    script = tmp_path / "w.py"
    script.write_text(
        "import sys, os\n"
        "sys.path.insert(0, %r)\n"
        "import torch, torch.distributed as dist\n"
        "from open_transformers_b200.parallel.env import init_distributed, shutdown_distributed\n"
        "rank, world, dev = init_distributed('cpu', timeout_s=60)\n"
        "t = torch.tensor([float(rank + 1)])\n"
        "dist.all_reduce(t)\n"
        "assert t.item() == 3.0 and world == 2 and dev.type == 'cpu'\n"
        "shutdown_distributed()\n"
        "print('ok', rank)\n" % str(ROOT))
    env = {k: v for k, v in os.environ.items() if k not in ("MASTER_ADDR", "MASTER_PORT")}
    if how == "tcp_store":
        env.update(DIST_MASTER_FQDN="127.0.0.1", DIST_MASTER_STORE_PORT=str(free_port()))
    else:
        env.update(TORCH_DIST_STORE_FILE=str(tmp_path / "store"))
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(2)]
    outs = [p.communicate(timeout=120)[0].decode() for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)[-3000:]


# ------------------------------------------------------------------ bounded device-side waits (one GPU, no peer involved)
def _cuda():
    import ctypes

    import torch

    from open_transformers_b200.ops.native import cuda_lib

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return ctypes, torch, cuda_lib()


@pytest.mark.gpu
def test_a_flag_wait_that_runs_out_reports_the_word_and_returns():
    """The wait that holds a bucket's gradient reduction until every rank has signalled it: five milliseconds, a word
    nothing writes. Status word 0 takes the caller's code, word 1 the index of the flag, and the stream goes on."""
    ctypes, torch, lib = _cuda()
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    flags[4] = 7                                     # rank 0 of bucket 2 (two ranks) has signalled epoch 7, rank 1 never does
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    t0 = time.time()
    rc = lib.otb_flag_wait(ctypes.c_void_p(flags.data_ptr()), ctypes.c_int(4), ctypes.c_int(2), ctypes.c_uint(7),
                           ctypes.c_ulonglong(5_000_000), ctypes.c_void_p(status.data_ptr()), ctypes.c_uint(4),
                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    after = torch.ones(8, device="cuda") * 3         # queued behind the wait on the same stream
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert status[:2].tolist() == [4, 5] and float(after.sum()) == 24.0
    # the same wait with both words set returns at once and leaves the status alone
    flags[5] = 7
    status.zero_()
    lib.otb_flag_wait(ctypes.c_void_p(flags.data_ptr()), ctypes.c_int(4), ctypes.c_int(2), ctypes.c_uint(7), ctypes.c_ulonglong(5_000_000),
                      ctypes.c_void_p(status.data_ptr()), ctypes.c_uint(4), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]


@pytest.mark.gpu
def test_a_peer_barrier_whose_peer_never_arrives_gives_status_3_and_a_late_row_block_gives_status_2():
    """`otb_peer_barrier` as rank 0 of 2 with a second slot array that no second rank exists to write, and
    `otb_tp_finish` on a result buffer whose arrival flags stay clear; both with the wait budget set to 5 ms."""
    ctypes, torch, lib = _cuda()
    lib.otb_set_peer_wait_ns.argtypes = [ctypes.c_ulonglong]
    assert lib.otb_set_peer_wait_ns(5_000_000) == 0
    try:
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        slots = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
        arr = (ctypes.c_void_p * 2)(slots[0].data_ptr(), slots[1].data_ptr())
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        assert lib.otb_peer_barrier(arr, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_uint(1), ctypes.c_void_p(status.data_ptr()), stream) == 0
        torch.cuda.synchronize()
        assert int(status[0]) == 3
        assert int(slots[0][0]) == 1 and int(slots[1][0]) == 1 and int(slots[0][1]) == 0   # it announced itself; nobody answered

        M = N = 128
        acc = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        tile_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        y = torch.full((M, N), 5.0, dtype=torch.bfloat16, device="cuda")
        status.zero_()
        rc = lib.otb_tp_finish(ctypes.c_void_p(acc.data_ptr()), ctypes.c_void_p(tile_flags.data_ptr()), ctypes.c_uint(1), ctypes.c_void_p(0),
                               ctypes.c_void_p(y.data_ptr()), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(0), ctypes.c_int(1),
                               ctypes.c_long(N), ctypes.c_long(N), ctypes.c_long(N), ctypes.c_void_p(status.data_ptr()), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status[0]) == 2 and bool((y == 5.0).all())   # no row block was delivered, none was written
    finally:
        assert lib.otb_set_peer_wait_ns(2_000_000_000) == 0
    assert float((torch.ones(4, device="cuda") + 1).sum()) == 8.0
