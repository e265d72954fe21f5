"""Failure detection, all on the host with CPU (gloo) ranks: a rank that leaves between steps is noticed by the
heartbeat before the survivor's next collective; a rank that never joins ends the rendezvous with an error after the
configured timeout; SIGTERM produces an off-cadence checkpoint whose hash replays; run-id disagreement and a missing
per-rank file are loud. No GPU is involved and nothing here makes a device fault, trap or hang."""
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

    def fake(world, device):
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
