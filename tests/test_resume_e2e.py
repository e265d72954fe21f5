"""Resume through the real train loop: a run that stops and is resumed from its checkpoint writes the hashes of the
uninterrupted run (weights, moments, optimizer step, data stream position, batch-hash chains, spike state and chained
hash all survive); a resumed run with a changed recipe is audited across the resume boundary with the old run's
checkpoint as the state and the new run's first checkpoint as the descriptor.
(reference test strategy: tests/e2e/test_100m_one_step.py, tests/distributed/test_checkpoint_resume_invariants.py)"""
import json
import shutil
from pathlib import Path

import pytest

from helpers import tiny_cfg
from open_transformers_b200.cli.audit_replay import AuditError, audit_replay
from open_transformers_b200.train.checkpoint import Checkpointer
from open_transformers_b200.train.loop import train

LONG = ["train.total_tokens=1280", "train.ckpt_every_steps=2"]  # 5 optimizer steps of 256 tokens


@pytest.fixture(scope="module")
def runs(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("resume"))
    whole = train(tiny_cfg(tmp, LONG + ["run.run_id=whole"]), device="cpu", data_root=tmp)
    first = train(tiny_cfg(tmp, LONG + ["run.run_id=parts"]), device="cpu", data_root=tmp, max_steps=2)
    return tmp, whole, first


def test_resumed_run_writes_the_uninterrupted_hashes(runs):
    tmp, whole, first = runs
    assert [s for s, _ in whole["hashes"]] == [1, 2, 3, 4, 5]
    assert first["hashes"] == whole["hashes"][:2]
    ck = first["run_dir"] + "/checkpoints/step_000000002"
    second = train(tiny_cfg(tmp, LONG + ["run.run_id=parts"]), resume_from=ck, device="cpu", data_root=tmp)
    assert second["hashes"] == whole["hashes"][2:]
    assert second["losses"] == whole["losses"][2:]
    meta = Checkpointer.read_meta(first["run_dir"] + "/checkpoints/step_000000004")
    assert meta.restart_count == 1 and meta.step == 4 and meta.chained_hash == dict(whole["hashes"])[4]
    rows = [json.loads(l) for l in open(first["run_dir"] + "/logs/state_hashes.jsonl")]
    assert [r["step"] for r in rows] == [0, 1, 2, 3, 4, 5]


def test_resume_with_a_reset_optimizer_forks_the_run(runs, tmp_path):
    tmp, whole, first = runs
    src = Path(first["run_dir"]) / "checkpoints" / "step_000000002"
    dst = tmp_path / "runs" / "fork" / "checkpoints" / "step_000000002"
    shutil.copytree(src, dst)
    cfg = tiny_cfg(tmp, LONG + ["run.run_id=fork", "run.output_dir=%s/runs" % tmp_path, "++train.resume_reset_optimizer=true"])
    forked = train(cfg, resume_from=str(dst), device="cpu", data_root=tmp, max_steps=3)
    assert forked["hashes"][0][0] == 3 and forked["hashes"][0][1] != dict(whole["hashes"])[3]


def test_resume_boundary_is_audited_with_the_new_runs_descriptor(runs, tmp_path):
    """the interval after a resume was trained by the resumed run's recipe: state from the old checkpoint, descriptor
    (configuration, topology) from the resumed run's first checkpoint"""
    tmp, whole, first = runs
    old = first["run_dir"] + "/checkpoints/step_000000002"
    new_cfg = tiny_cfg(tmp, LONG + ["run.run_id=fixed", "run.output_dir=%s/runs" % tmp_path, "train.grad_clip=0.05"])
    fixed = train(new_cfg, resume_from=old, device="cpu", data_root=tmp)
    new_first = fixed["run_dir"] + "/checkpoints/step_000000004"
    want = dict(fixed["hashes"])[4]
    assert want != dict(whole["hashes"])[4]                      # the changed clip really changed the run
    ok = audit_replay(old, descriptor_checkpoint=new_first, data_root=tmp, until_step=4, expect_hash=new_first + "/state_hash.txt")
    assert ok["match"] is True and ok["state_hash"] == want
    stale = audit_replay(old, data_root=tmp, until_step=4, expect_hash=want)   # the old run's own descriptor
    assert stale["match"] is False and stale["state_hash"] == dict(whole["hashes"])[4]
    # a descriptor from another lineage (different seed) is refused
    other = train(tiny_cfg(tmp, LONG + ["run.run_id=other", "run.output_dir=%s/runs" % tmp_path, "run.seed=7"]), device="cpu", data_root=tmp, max_steps=2)
    with pytest.raises(AuditError):
        audit_replay(old, descriptor_checkpoint=other["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=4)


WORKER = """
import json, os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
from helpers import tiny_cfg
from open_transformers_b200.train.loop import train
from open_transformers_b200.parallel.env import shutdown_distributed
cfg = tiny_cfg({tmp!r}, {extra!r})
res = train(cfg, resume_from={resume!r}, device="cpu", data_root={tmp!r}, max_steps={max_steps!r})
if int(os.environ["RANK"]) == 0:
    json.dump(res["hashes"], open({out!r}, "w"))
shutdown_distributed()
"""


def _ranks(n, tmp, extra, resume, max_steps, out, **env_extra):
    import os
    import subprocess
    import sys

    from helpers import free_port

    root = str(Path(__file__).resolve().parent.parent)
    script = Path(out + ".py")
    script.write_text(WORKER.format(root=root, tmp=tmp, extra=extra, resume=resume, max_steps=max_steps, out=out))
    port = free_port()
    procs = [subprocess.Popen([sys.executable, str(script)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              env=dict(os.environ, RANK=str(r), WORLD_SIZE=str(n), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                                       MASTER_PORT=str(port), OMP_NUM_THREADS="2", **env_extra)) for r in range(n)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=300)[0].decode())
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)[-5000:]
    return [tuple(x) for x in json.load(open(out))]


@pytest.mark.distributed
def test_a_run_resumes_on_a_different_number_of_processes(runs, tmp_path):
    """the virtual topology, not the process count, defines the run: two processes write the checkpoint, one process
    resumes it (and the other way round), and the hashes are those of the uninterrupted single-process run"""
    tmp, whole, first = runs
    base = LONG + ["run.output_dir=%s/runs" % tmp_path]
    two = _ranks(2, tmp, base + ["run.run_id=g2"], None, 2, str(tmp_path / "g2_first.json"))
    assert two == whole["hashes"][:2]
    ck = "%s/runs/g2/checkpoints/step_000000002" % tmp_path
    for f in ("rng.rank_0.pt", "rng.rank_1.pt", "batch_hasher.rank_0.bin", "batch_hasher.rank_1.bin"):
        assert (Path(ck) / f).exists(), f                          # one file per VIRTUAL rank, whoever hosted it
    one = train(tiny_cfg(tmp, base + ["run.run_id=g2"]), resume_from=ck, device="cpu", data_root=tmp)
    assert one["hashes"] == whole["hashes"][2:]
    # and a single-process checkpoint resumed by two processes
    back = _ranks(2, tmp, base + ["run.run_id=g1to2"], first["run_dir"] + "/checkpoints/step_000000002", None, str(tmp_path / "g1to2.json"))
    assert back == whole["hashes"][2:]


def test_off_cadence_final_checkpoint_hash_equals_log_and_replay_and_does_not_advance_the_chain(tmp_path):
    """hash every 2 steps, run of 3 steps: the final checkpoint's hash is computed off the cadence; it is the logged one and
    the replayed one, and the chain a resumed run continues from is still the step-2 hash
    (reference tests/e2e/test_final_emergency_ckpt_hash.py:135-178)"""
    tmp = str(tmp_path)
    over = ["train.state_hash.every_n_steps=2", "train.ckpt_every_steps=100", "train.total_tokens=1280"]
    short = train(tiny_cfg(tmp, over + ["run.run_id=short"]), device="cpu", data_root=tmp, max_steps=3)
    assert [s for s, _ in short["hashes"]] == [2, 3]
    ck = Path(short["run_dir"]) / "checkpoints" / "step_000000003"
    final = (ck / "state_hash.txt").read_text().strip()
    rows = [json.loads(l) for l in open(short["run_dir"] + "/logs/state_hashes.jsonl")]
    assert rows[-1]["step"] == 3 and rows[-1]["state_hash"] == final == dict(short["hashes"])[3]
    meta = Checkpointer.read_meta(ck)
    assert meta.chained_hash == dict(short["hashes"])[2]                                                        # not the off-cadence one
    r = audit_replay(from_init=True, descriptor_checkpoint=str(ck), data_root=tmp, until_step=3, expect_hash=final)
    assert r["match"] is True
    # a longer run with the same cadence, and the short run resumed to the same length, agree on the step-4 hash
    long_over = over
    whole = train(tiny_cfg(tmp, long_over + ["run.run_id=long"]), device="cpu", data_root=tmp)
    resumed = train(tiny_cfg(tmp, long_over + ["run.run_id=short"]), resume_from=str(ck), device="cpu", data_root=tmp)
    assert dict(resumed["hashes"])[4] == dict(whole["hashes"])[4] and dict(resumed["hashes"])[5] == dict(whole["hashes"])[5]


@pytest.mark.distributed
@pytest.mark.parametrize("packed", [False, True])
def test_sharded_ownership_by_messages_through_the_train_loop_and_a_checkpoint(tmp_path, packed):
    """two processes with sharded ownership over point-to-point messages (the transport of GPUs on several machines): hashes
    of the single-process run, a checkpoint into which each process wrote the rows it owns (data files of both processes,
    no gathering to rank 0), and a single-process resume from it. ``packed``: run.state_sharding, where each process holds
    the moments of its own segments only - the checkpoint is the same, and two such processes resume from it too"""
    tmp = str(tmp_path)
    over = LONG + ["++train.state_hash.tensor_digest=tree"]
    whole = train(tiny_cfg(tmp, over + ["run.run_id=one"]), device="cpu", data_root=tmp)
    shard = ["run.state_sharding=true"] if packed else []
    two = _ranks(2, tmp, over + shard + ["run.run_id=msg"], None, 2, str(tmp_path / "msg.json"), OTB_GRAD_TRANSPORT="collective")
    assert two == whole["hashes"][:2]
    if packed:
        again = _ranks(2, tmp, over + shard + ["run.run_id=msg2"], "%s/runs/msg/checkpoints/step_000000002" % tmp, None, str(tmp_path / "msg2.json"),
                       OTB_GRAD_TRANSPORT="collective")
        assert again == whole["hashes"][2:]
    files = sorted(p.name for p in Path("%s/runs/msg/checkpoints/step_000000002/dcp" % tmp).iterdir())
    assert ".metadata" in files and any(f.startswith("__0_") for f in files) and any(f.startswith("__1_") for f in files), files
    rest = train(tiny_cfg(tmp, over + ["run.run_id=msg"]), resume_from="%s/runs/msg/checkpoints/step_000000002" % tmp, device="cpu", data_root=tmp)
    assert rest["hashes"] == whole["hashes"][2:]


def test_replay_loss_log_equals_the_training_metrics_bit_for_bit(runs, tmp_path):
    """--loss-log: the replay's per-step mean loss and gradient norm are the numbers the trainer logged, exactly"""
    tmp, whole, first = runs
    log = tmp_path / "losses.jsonl"
    r = audit_replay(from_init=True, descriptor_checkpoint=whole["run_dir"] + "/checkpoints/step_000000004", data_root=tmp, until_step=4,
                     loss_log=str(log))
    assert r["match"] is True
    mine = [json.loads(l) for l in log.read_text().splitlines()]
    theirs = [json.loads(l) for l in open(whole["run_dir"] + "/logs/metrics.jsonl")][:4]
    assert [m["step"] for m in mine] == [1, 2, 3, 4]
    assert [m["loss"] for m in mine] == [t["loss"] for t in theirs]
    assert [m["grad_norm"] for m in mine] == [t["grad_norm_pre_clip"] for t in theirs]
    # the tensor-level diagnostic: against the checkpoint of the replayed step nothing differs, against an earlier one everything does
    import os

    ck4, ck2 = whole["run_dir"] + "/checkpoints/step_000000004", whole["run_dir"] + "/checkpoints/step_000000002"
    for env_name, against, want_zero in (("PRETRAIN_AUDIT_DIFF_CKPT", ck4, True), ("REPOP_AUDIT_DIFF_CKPT", ck2, False)):
        os.environ[env_name] = against
        try:
            d = audit_replay(from_init=True, descriptor_checkpoint=ck4, data_root=tmp, until_step=4)["diff"]
        finally:
            del os.environ[env_name]
        assert d["tensors"] > 0 and (d["differing"] == 0) == want_zero and len(d["top"]) <= 15 and d["top"][0][1] in ("param", "optim.exp_avg", "optim.exp_avg_sq")
    # metrics.jsonl carries the reference's keys (src/pretrain/train/loop.py, metrics.log) beside this package's own
    wanted = {"consumed_tokens", "lr", "accum_steps", "grad_norm_pre_clip", "loss_ce", "loss_zloss", "perplexity", "loss_ce_global", "loss_zloss_global",
              "perplexity_global", "tokens_per_sec", "tokens_per_sec_per_gpu", "mfu", "step_compute_time_ms", "step_wall_time_ms", "hash_time_ms",
              "ckpt_save_time_ms", "skipped_steps_total"}
    assert wanted <= set(theirs[0]) and theirs[0]["loss_ce_global"] == theirs[0]["loss"] and theirs[0]["step_compute_time_ms"] <= theirs[0]["step_wall_time_ms"]


def test_skipped_steps_are_replayed_as_skips_and_a_halt_ends_the_run(tmp_path):
    """spike protocol through the loop: with a threshold below every gradient norm every step from ``start_step`` on is
    skipped (a fresh spike, then its cool-down skip, alternately): weights stay untouched while data is consumed, and the
    replay takes the same decisions, from the seed and from a checkpoint taken inside a cool-down; with a shorter cool-down
    the fresh spikes reach the halt count and the run stops"""
    tmp = str(tmp_path)
    over = LONG + ["train.spike.grad_norm_threshold=0.0001", "train.spike.skip_steps_on_spike=2", "train.spike.skips_in_window_to_halt=3",
                   "train.spike.halt_window_steps=100", "train.spike.start_step=1"]
    res = train(tiny_cfg(tmp, over + ["run.run_id=spiky"]), device="cpu", data_root=tmp)
    rows = [json.loads(l) for l in open(res["run_dir"] + "/logs/metrics.jsonl")]
    skipped = [r["skipped"] for r in rows]
    assert skipped == [False, True, True, True, True], skipped                       # the first step is before start_step
    assert rows[-1]["skipped_steps_total"] == 4 and "halted" not in res                # fresh spikes at steps 1 and 3 only: below the halt count
    from open_transformers_b200.cli.hash_ckpt import hash_checkpoint

    assert hash_checkpoint(res["run_dir"] + "/checkpoints/step_000000002", include_optimizer=False) == \
        hash_checkpoint(res["run_dir"] + "/checkpoints/step_000000004", include_optimizer=False)   # no update in between
    ck = res["run_dir"] + "/checkpoints/step_000000004"
    r = audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=4)
    assert r["match"] is True
    r = audit_replay(res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=4)     # spike state restored from the checkpoint
    assert r["match"] is True
    calm = train(tiny_cfg(tmp, LONG + ["run.run_id=calm"]), device="cpu", data_root=tmp)
    assert dict(calm["hashes"])[4] != dict(res["hashes"])[4]
    halting = over[:-4] + ["train.spike.skip_steps_on_spike=1", "train.spike.skips_in_window_to_halt=2", "train.spike.halt_window_steps=100",
                           "train.spike.start_step=0"]
    halted = train(tiny_cfg(tmp, halting + ["run.run_id=halts"]), device="cpu", data_root=tmp)
    assert "halted" in halted and halted["step"] < 5


def test_batch_size_phase_change_mid_run_trains_replays_and_resumes(tmp_path):
    """the global batch doubles after 512 tokens (two micro-batches per virtual rank instead of one): trained, replayed from
    the seed across the change, and resumed from the checkpoint that sits on it"""
    tmp = str(tmp_path)
    over = ["train.total_tokens=2048", "train.ckpt_every_steps=2", "train.global_batch_tokens.warmup=256", "train.global_batch_tokens.main=512",
            "train.global_batch_tokens.late=512", "train.warmup_to_main_at_tokens=512", "train.main_to_late_at_tokens=100000"]
    res = train(tiny_cfg(tmp, ["run.run_id=phases"] + over), device="cpu", data_root=tmp)
    rows = [json.loads(l) for l in open(res["run_dir"] + "/logs/metrics.jsonl")]
    assert [r["microbatches"] for r in rows] == [2, 2, 4, 4, 4] and [r["consumed_tokens"] for r in rows] == [256, 512, 1024, 1536, 2048]
    ck4 = res["run_dir"] + "/checkpoints/step_000000004"
    assert audit_replay(from_init=True, descriptor_checkpoint=ck4, data_root=tmp, until_step=4)["match"] is True
    ck2 = res["run_dir"] + "/checkpoints/step_000000002"
    assert audit_replay(ck2, data_root=tmp, until_step=4)["match"] is True
    first = train(tiny_cfg(tmp, ["run.run_id=phases2"] + over), device="cpu", data_root=tmp, max_steps=2)
    rest = train(tiny_cfg(tmp, ["run.run_id=phases2"] + over), resume_from=first["run_dir"] + "/checkpoints/step_000000002", device="cpu", data_root=tmp)
    assert first["hashes"] + rest["hashes"] == res["hashes"]


def test_rewarm_after_a_resume_is_recorded_and_replayed(runs, tmp_path):
    """schedule.rewarm_on_resume: the resumed run ramps the learning rate from zero over ``rewarm_tokens``, anchored at the
    resume point; the anchor travels in the resumed run's checkpoints, so the boundary interval replays with them as
    descriptor"""
    tmp, whole, first = runs
    old = first["run_dir"] + "/checkpoints/step_000000002"
    cfg = tiny_cfg(tmp, LONG + ["run.run_id=rewarm", "run.output_dir=%s/runs" % tmp_path, "++schedule.rewarm_on_resume=true", "++schedule.rewarm_tokens=512"])
    res = train(cfg, resume_from=old, device="cpu", data_root=tmp)
    rows = [json.loads(l) for l in open(res["run_dir"] + "/logs/metrics.jsonl")]
    base = {r["step"]: r["lr"] for r in (json.loads(l) for l in open(whole["run_dir"] + "/logs/metrics.jsonl"))}
    assert [r["step"] for r in rows] == [3, 4, 5]
    assert rows[0]["lr"] == 0.0 and rows[1]["lr"] == pytest.approx(0.5 * base[4]) and rows[2]["lr"] == pytest.approx(base[5])
    new_first = res["run_dir"] + "/checkpoints/step_000000004"
    assert Checkpointer.read_meta(new_first).rewarm_anchor_tokens == 512
    r = audit_replay(old, descriptor_checkpoint=new_first, data_root=tmp, until_step=4, expect_hash=dict(res["hashes"])[4])
    assert r["match"] is True and dict(res["hashes"])[4] != dict(whole["hashes"])[4]


@pytest.mark.parametrize("extra", [["++train.state_hash.include_grads=false"], ["++train.state_hash.include_batch=false"],
                                   ["++train.state_hash.tensor_digest=tree", "++train.state_hash.include_grads=false", "++train.state_hash.include_batch=false"],
                                   ["model.modules.attention=gqa_qknorm_repop", "model.qk_norm=true", "model.qk_norm_gain=true", "++train.qk_gain_clamp=1.0001",
                                    "++train.qk_freeze_q_gains_until_step=2"]])
def test_hash_content_switches_and_gain_controls_replay(tmp_path, extra):
    """what the state hash covers (gradients, batch digest, raw bytes or tree digests) and the QK-gain controls (clamp
    after the update, query gains frozen for the first steps) are part of the recipe: the replay follows them"""
    tmp = str(tmp_path)
    res = train(tiny_cfg(tmp, ["train.ckpt_every_steps=2", *extra]), device="cpu", data_root=tmp)
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    assert audit_replay(ck, data_root=tmp, until_step=3)["match"] is True
    assert audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=3)["match"] is True
    plain = train(tiny_cfg(tmp + "/p", ["train.ckpt_every_steps=2"]), device="cpu", data_root=tmp + "/p")
    assert plain["hashes"][-1][1] != res["hashes"][-1][1]


def test_token_clocked_checkpoints_and_latest(tmp_path):
    """train.ckpt_every_tokens (with ckpt_every_steps = 0): a checkpoint whenever the consumed-token count crosses a multiple,
    plus the final one; ``latest`` finds the newest complete one and ignores a half-written directory"""
    tmp = str(tmp_path)
    res = train(tiny_cfg(tmp, LONG + ["train.ckpt_every_steps=0", "train.ckpt_every_tokens=512"]), device="cpu", data_root=tmp)
    ckdir = Path(res["run_dir"]) / "checkpoints"
    assert sorted(p.name for p in ckdir.glob("step_*")) == ["step_000000002", "step_000000004", "step_000000005"]
    ck = Checkpointer(res["run_dir"])
    assert ck.complete_steps() == [2, 4, 5] and Path(ck.latest()).name == "step_000000005"
    (ckdir / "step_000000005" / "_COMPLETE").unlink()              # a writer that died before finishing
    assert Path(ck.latest()).name == "step_000000004"
    r = audit_replay(str(ckdir / "step_000000002"), data_root=tmp)  # default span: to the next checkpoint of the cadence
    assert r["step"] == 4 and r["match"] is True


def test_the_tensor_payload_is_what_a_torch_optimizer_and_module_would_save(runs):
    """dcp/ holds {"model": state_dict, "optim": optimizer.state_dict()} in torch's own packing: optimizer state under
    integer parameter indices (numbered group by group) and a `params` index list in every param_group. A plain module
    with the same parameter names and a torch.optim.Optimizer over the same [decay, no_decay] groups provide the template;
    DCP fills it and the values are the engine's."""
    import torch
    import torch.distributed.checkpoint as dcp

    from open_transformers_b200.train.checkpoint import Checkpointer
    from open_transformers_b200.train.engine import TrainEngine

    tmp, whole, first = runs
    ck = whole["run_dir"] + "/checkpoints/step_000000004"
    cfg = tiny_cfg(tmp, LONG)
    eng = TrainEngine(cfg, "cpu")
    Checkpointer(whole["run_dir"]).load(ck, eng)
    lay = eng.layout
    params = {n: torch.nn.Parameter(torch.zeros(lay.shapes[i])) for i, n in enumerate(lay.names)}
    groups = [{"params": [params[n] for n, m in zip(lay.names, lay.groups) if m == gi], "weight_decay": g["weight_decay"]}
              for gi, g in enumerate(eng.param_groups)]
    class Shell(torch.optim.Optimizer):               # the reference's optimizer shell: these defaults, state per parameter
        def __init__(self, groups):
            super().__init__(groups, dict(lr=1.0, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, amsgrad=False))

    opt = Shell(groups)
    for p in params.values():                         # primed state, as prime_optimizer_state leaves it
        opt.state[p] = {"step": torch.zeros((), dtype=torch.int64), "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
    template = {"model": {n: p.data for n, p in params.items()}, "optim": opt.state_dict()}
    dcp.load(template, storage_reader=dcp.FileSystemReader(ck + "/dcp"), no_dist=True)
    opt.load_state_dict(template["optim"])
    for i, n in enumerate(lay.names):
        st = opt.state[params[n]]
        assert torch.equal(params[n].data, lay.view(eng.master, i)), n
        assert torch.equal(st["exp_avg"], lay.view(eng.m1, i)) and torch.equal(st["exp_avg_sq"], lay.view(eng.m2, i)), n
        assert int(st["step"]) == eng.opt_step == 4
    assert [g["lr"] for g in opt.param_groups] == [g["lr"] for g in eng.param_groups]
    eng.close()
