"""End to end on the CPU: the real ``train()`` on a tiny decoder, then the real audit replay, hand-off
verification, safetensors relay, and the same run on two gloo ranks (its hashes must equal the single-process
run: the virtual topology, not the process count, defines the bytes)."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from helpers import free_port, tiny_cfg
from open_transformers_b200.cli.audit_replay import audit_replay, main as audit_main, resolve_expect_hash
from open_transformers_b200.cli.dcp_safetensors import pack, unpack
from open_transformers_b200.cli.hash_ckpt import hash_checkpoint
from open_transformers_b200.cli.verify_handoff import verify_handoff
from open_transformers_b200.train.loop import train

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("run"))
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=2"])
    res = train(cfg, device="cpu", data_root=tmp)
    return tmp, cfg, res


def test_train_writes_the_run_directory(trained):
    tmp, cfg, res = trained
    run = Path(res["run_dir"])
    assert [s for s, _ in res["hashes"]] == [1, 2, 3] and len({h for _, h in res["hashes"]}) == 3
    rows = [json.loads(l) for l in (run / "logs" / "state_hashes.jsonl").read_text().splitlines()]
    assert rows[0]["kind"] == "init" and [r["step"] for r in rows[1:]] == [1, 2, 3]
    assert (run / "checkpoints" / "state_hash_init.txt").read_text().strip() == rows[0]["state_hash"]
    for step in (2, 3):
        d = run / "checkpoints" / ("step_%09d" % step)
        for f in ("_COMPLETE", "meta.json", "state_hash.txt", "global_stream.json", "spike_protocol.json", "batch_hasher.rank_0.bin",
                  "batch_hasher.rank_1.bin", "rng.rank_0.pt", "rng.rank_1.pt", "dcp/.metadata"):
            assert (d / f).exists(), f
        assert len((d / "batch_hasher.rank_1.bin").read_bytes()) == 32
    metrics = [json.loads(l) for l in (run / "logs" / "metrics.jsonl").read_text().splitlines()]
    assert len(metrics) == 3 and all(m["loss"] > 0 for m in metrics)


def test_cold_start_guard_refuses_to_overwrite(trained):
    tmp, cfg, res = trained
    with pytest.raises(RuntimeError):
        train(cfg, device="cpu", data_root=tmp)


def test_replay_from_init_and_from_checkpoint_match(trained):
    tmp, cfg, res = trained
    final = res["hashes"][-1][1]
    r = audit_replay(from_init=True, descriptor_checkpoint=res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3)
    assert r["init_match"] is True and r["match"] is True and r["state_hash"] == final
    assert r["kernels"] == ["otb_cpu"] and len(r["build"]["native_source_digests"]["otb_cpu"]) == 64 and r["build"]["git_sha"]
    r2 = audit_replay(res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3, expect_hash=final)
    assert r2["match"] is True and len(r2["rank0_losses"]) == 1
    bad = audit_replay(res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3, expect_hash="0" * 64)
    assert bad["match"] is False


def test_cli_exit_codes_and_messages(trained, capsys):
    tmp, cfg, res = trained
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    assert audit_main(["--checkpoint", ck, "--data-root", tmp, "--until-step", "3"]) == 0
    assert "MATCH=True" in capsys.readouterr().out
    assert audit_main(["--checkpoint", ck, "--data-root", tmp, "--until-step", "3", "--expect-hash", "f" * 64]) == 1
    assert "AUDIT FAILED: state_hash" in capsys.readouterr().err
    assert audit_main(["--checkpoint", ck, "--data-root", tmp, "--until-step", "1"]) == 2
    with pytest.raises(Exception):
        resolve_expect_hash("not-a-digest")


def test_tampered_checkpoint_is_detected(trained, tmp_path):
    tmp, cfg, res = trained
    import shutil

    import torch

    src = Path(res["run_dir"]) / "checkpoints" / "step_000000002"
    dst = tmp_path / "checkpoints" / "step_000000002"
    shutil.copytree(src, dst)
    chain = bytearray((dst / "batch_hasher.rank_0.bin").read_bytes())
    chain[0] ^= 1
    (dst / "batch_hasher.rank_0.bin").write_bytes(bytes(chain))
    r = audit_replay(str(dst), data_root=tmp, until_step=3, expect_hash=res["hashes"][-1][1])
    assert r["match"] is False
    (dst / "rng.rank_1.pt").unlink()
    with pytest.raises(FileNotFoundError):
        audit_replay(str(dst), data_root=tmp, until_step=3)


def test_handoff_and_safetensors_relay(trained, tmp_path):
    tmp, cfg, res = trained
    ck2 = res["run_dir"] + "/checkpoints/step_000000002"
    packed = pack(ck2, str(tmp_path / "ck.safetensors"))
    assert packed["tensors"] > 0
    un = unpack(str(tmp_path / "ck.safetensors"), str(tmp_path / "relay" / "checkpoints" / "step_000000002"))
    assert hash_checkpoint(un["dir"]) == hash_checkpoint(ck2)
    r = audit_replay(un["dir"], data_root=tmp, until_step=3, save_checkpoint_dir=str(tmp_path / "handoff"), expect_hash=res["hashes"][-1][1])
    assert r["match"] is True
    prev = dict(res["hashes"])[2]
    want = dict(res["hashes"])[3]
    v = verify_handoff(r["saved_checkpoint"], expect_hash=want, prev_hash=prev)
    assert v["verified"] is True and v["reconstructed_hash"] == want
    assert verify_handoff(r["saved_checkpoint"], expect_hash=want, prev_hash="1" * 64)["verified"] is False


WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
    from helpers import tiny_cfg
    from open_transformers_b200.train.loop import train
    from open_transformers_b200.parallel.env import shutdown_distributed
    cfg = tiny_cfg({tmp!r}, ["run.run_id={run_id}", "train.ckpt_every_steps=2", "run.tp_size={tp}"])
    res = train(cfg, device="cpu", data_root={tmp!r})
    if int(os.environ["RANK"]) == 0:
        json.dump(res["hashes"], open({tmp!r} + "/{run_id}_hashes.json", "w"))
    shutdown_distributed()
""")


def _two_ranks(tmp, run_id, tp):
    script = Path(tmp) / ("worker_%s.py" % run_id)
    script.write_text(WORKER.format(root=str(ROOT), tmp=tmp, run_id=run_id, tp=tp))
    port = free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out.decode())
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    return [tuple(x) for x in json.load(open(tmp + "/%s_hashes.json" % run_id))]


@pytest.mark.distributed
def test_two_gloo_ranks_produce_the_single_process_hashes(trained):
    tmp, cfg, res = trained
    assert _two_ranks(tmp, "dist", 1) == [tuple(x) for x in res["hashes"]]
    # and the two-rank run's checkpoint replays on one process
    r = audit_replay(tmp + "/runs/dist/checkpoints/step_000000002", data_root=tmp, until_step=3)
    assert r["match"] is True


@pytest.mark.distributed
def test_a_tensor_parallel_pair_trains_to_the_single_process_hashes(trained):
    """The real ``train()`` with run.tp_size = 2 on two gloo ranks: same hash log as the unsplit run, and its checkpoint
    (written by a tensor-parallel run) replays unsplit on one process."""
    tmp, cfg, res = trained
    assert _two_ranks(tmp, "tp2", 2) == [tuple(x) for x in res["hashes"]]
    r = audit_replay(tmp + "/runs/tp2/checkpoints/step_000000002", data_root=tmp, until_step=3)
    assert r["match"] is True


def test_replay_with_folded_gradients_and_verified_spill(trained, tmp_path):
    """--offload-grads (one work buffer + one partial per replica) and --fold-spill-dir give the very digests of the plain
    replay; a spilled partial that was tampered with is refused."""
    from open_transformers_b200.train.engine import SpillCorruption, TrainEngine

    tmp, cfg, res = trained
    ck = tmp + "/runs/t/checkpoints/step_000000002"
    plain = audit_replay(ck, data_root=tmp, until_step=3)
    folded = audit_replay(ck, data_root=tmp, until_step=3, offload_grads=True)
    spilled = audit_replay(ck, data_root=tmp, until_step=3, offload_grads=True, fold_spill_dir=str(tmp_path / "spill"))
    assert plain["match"] and folded["match"] and spilled["match"]
    assert plain["state_hash"] == folded["state_hash"] == spilled["state_hash"]
    assert (tmp_path / "spill" / "replica_000.f32.blake2b").exists()
    # corruption of a spilled partial
    eng = TrainEngine(cfg, "cpu", fold_gradients=True, fold_spill_dir=str(tmp_path / "spill2"))
    eng.zero_grads()
    for v in range(eng.V):
        eng.fold_virtual_rank(v)
    path = tmp_path / "spill2" / "replica_000.f32"
    raw = bytearray(path.read_bytes())
    raw[5] ^= 1
    path.write_bytes(bytes(raw))
    with pytest.raises(SpillCorruption):
        eng.reduce_gradients()
    eng.close()


def test_folded_replay_with_gradient_accumulation_matches_the_plain_replay(tmp_path):
    """Two micro-batches per virtual rank: the loader hands them out interleaved (v0k0, v1k0, v0k1, v1k1); the folded
    replay has one work buffer and must run rank by rank. Its digests equal the run's and the plain replay's."""
    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=1", "train.global_batch_tokens.warmup=512", "train.global_batch_tokens.main=512",
                         "train.global_batch_tokens.late=512", "train.total_tokens=1024"])
    mb_tokens = cfg.train.micro_batch_size * cfg.train.seq_len * cfg.run.virtual_dp_size
    assert 512 // mb_tokens >= 2, "the recipe must accumulate at least two micro-batches per virtual rank"
    res = train(cfg, device="cpu", data_root=tmp)
    ck = res["run_dir"] + "/checkpoints/step_000000001"
    plain = audit_replay(ck, data_root=tmp, until_step=2)
    folded = audit_replay(ck, data_root=tmp, until_step=2, offload_grads=True)
    assert plain["match"] is True and folded["match"] is True and plain["state_hash"] == folded["state_hash"] == res["hashes"][-1][1]


def test_replay_with_offloaded_moments_and_master(trained, tmp_path):
    """--offload-optimizer / --offload-master keep the moments and the fp32 master weights in files; the digests are
    those of the plain replay, from a checkpoint and from the initial state, and the files hold the final state."""
    import numpy as np

    tmp, cfg, res = trained
    ck = tmp + "/runs/t/checkpoints/step_000000002"
    plain = audit_replay(ck, data_root=tmp, until_step=4, save_checkpoint_dir=str(tmp_path / "plain"))
    od, md = tmp_path / "moments", tmp_path / "master"
    off = audit_replay(ck, data_root=tmp, until_step=4, offload_optimizer=True, optimizer_offload_dir=str(od),
                       offload_master=True, master_offload_dir=str(md), offload_grads=True, save_checkpoint_dir=str(tmp_path / "off"))
    assert plain["state_hash"] == off["state_hash"] and off["state_hash"] is not None
    assert {p.name for p in od.iterdir()} == {"exp_avg.bin", "exp_avg_sq.bin"} and (md / "master.bin").exists()
    m1 = np.fromfile(od / "exp_avg.bin", dtype=np.float32)
    assert np.isfinite(m1).all() and np.abs(m1).max() > 0 and np.fromfile(od / "exp_avg_sq.bin", dtype=np.float32).min() >= 0
    # temporary directories when none is named; from the initial state
    a = audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=2)
    b = audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=2, offload_optimizer=True, offload_master=True)
    assert a["match"] is True and b["match"] is True and a["state_hash"] == b["state_hash"]


def test_replay_with_the_streaming_vocabulary_head(trained, monkeypatch):
    """PRETRAIN_AUDIT_STREAM_HEAD=1: head and loss in row panels (here 48 rows of 128, so with a ragged last panel);
    the fp32 replay keeps every bit"""
    tmp, cfg, res = trained
    ck = tmp + "/runs/t/checkpoints/step_000000002"
    monkeypatch.setenv("PRETRAIN_AUDIT_STREAM_HEAD", "1")
    monkeypatch.setenv("PRETRAIN_AUDIT_HEAD_CHUNK_ROWS", "48")
    from open_transformers_b200.train import engine as E

    calls = []
    real = E.streaming_head_loss
    monkeypatch.setattr(E, "streaming_head_loss", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    r = audit_replay(ck, data_root=tmp, until_step=3)
    assert r["match"] is True and calls
    r0 = audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=2)
    assert r0["match"] is True
