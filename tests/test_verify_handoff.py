"""Hand-off verification from disk alone: a checkpoint saved by the replay carries its post-clip gradients; the verifier
rebuilds the published chained hash without a forward or backward pass, and refuses - with a reason - every artifact whose
hash it cannot honestly rebuild: altered tensors, gradients, batch chains or links, incomplete or foreign gradient files,
partial downloads, off-cadence checkpoints, self-contradicting claims, implausible topologies.
(reference test strategy: tests/test_verify_handoff.py, tests/test_audit_gradient_sidecar.py)"""
import json
import os
import shutil
from pathlib import Path

import pytest
import torch

from helpers import tiny_cfg
from open_transformers_b200.cli import verify_handoff as VH
from open_transformers_b200.cli.audit_replay import audit_replay
from open_transformers_b200.cli.verify_handoff import (HandoffError, main as verify_main, read_batch_digest, read_gradient_sidecar,
                                                       verify_handoff, write_gradient_sidecar)
from open_transformers_b200.train.loop import train


@pytest.fixture(scope="module")
def handoff(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("handoff"))
    res = train(tiny_cfg(tmp, ["train.ckpt_every_steps=2"]), device="cpu", data_root=tmp)
    out = tmp + "/relay"
    r = audit_replay(res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3, save_checkpoint_dir=out)
    assert r["match"] is True
    return tmp, res, r["saved_checkpoint"], dict(res["hashes"])


def _copy(src, dst):
    shutil.copytree(src, dst)
    return Path(dst)


def _edit_meta(d, **over):
    meta = json.loads((d / "meta.json").read_text())
    meta.update(over)
    (d / "meta.json").write_text(json.dumps(meta))


def test_a_downloaded_handoff_reproduces_the_published_hash(handoff):
    tmp, res, ck, hashes = handoff
    v = verify_handoff(ck, expect_hash=hashes[3], prev_hash=hashes[2])
    assert v["verified"] is True and v["reconstructed_hash"] == hashes[3] == v["expected_hash"] and v["step"] == 3
    assert v["dp_world_size"] == 2 and v["include_grads"] and v["include_batch"] and v["gradients_attached"] > 0
    # upper-case and padded literals are the same commitment
    assert verify_handoff(ck, expect_hash="  %s\n" % hashes[3].upper(), prev_hash=hashes[2])["verified"] is True


def test_the_wrong_preceding_or_target_commitment_fails(handoff, tmp_path):
    tmp, res, ck, hashes = handoff
    assert verify_handoff(ck, expect_hash=hashes[3], prev_hash=hashes[1])["verified"] is False
    # a wrong target that the artifact itself does not contradict (no state_hash.txt to compare with)
    d = _copy(ck, tmp_path / "t" / "checkpoints" / "step_000000003")
    (d / "state_hash.txt").unlink()
    v = verify_handoff(str(d), expect_hash="0" * 64, prev_hash=hashes[2])
    assert v["verified"] is False and v["reconstructed_hash"] == hashes[3]


def test_commitments_are_literal_digests_and_the_bad_flag_is_named(handoff, tmp_path):
    tmp, res, ck, hashes = handoff
    f = tmp_path / "hash.txt"
    f.write_text(hashes[3])
    for flag, kw in (("--expect-hash", dict(expect_hash=str(f), prev_hash=hashes[2])), ("--prev-hash", dict(expect_hash=hashes[3], prev_hash=str(f))),
                     ("--expect-hash", dict(expect_hash=hashes[3][:16], prev_hash=hashes[2])), ("--prev-hash", dict(expect_hash=hashes[3], prev_hash=""))):
        with pytest.raises(HandoffError, match=flag + " takes the 64 hex digits of a published hash"):
            verify_handoff(ck, **kw)


def test_sidecar_round_trip_keeps_absent_gradients_apart_from_zero_ones(tmp_path):
    g = {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "b": None, "c": torch.zeros(4)}
    write_gradient_sidecar(tmp_path, g)
    back = read_gradient_sidecar(tmp_path)
    assert set(back) == {"a", "b", "c"} and back["b"] is None and torch.equal(back["a"], g["a"]) and torch.equal(back["c"], g["c"])


def test_altered_state_fails_the_commitment(handoff, tmp_path):
    tmp, res, ck, hashes = handoff
    # one gradient element, one unit in the last place
    d = _copy(ck, tmp_path / "g" / "checkpoints" / "step_000000003")
    grads = read_gradient_sidecar(d)
    name = sorted(n for n, t in grads.items() if t is not None and t.numel() > 10)[0]
    grads[name].view(-1).view(torch.int32)[3] ^= 1
    write_gradient_sidecar(d, grads)
    assert verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])["verified"] is False
    # one bit of one rank's batch chain
    d = _copy(ck, tmp_path / "b" / "checkpoints" / "step_000000003")
    raw = bytearray((d / "batch_hasher.rank_1.bin").read_bytes())
    raw[31] ^= 0x80
    (d / "batch_hasher.rank_1.bin").write_bytes(bytes(raw))
    assert verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])["verified"] is False
    # the two ranks' chains swapped: same bytes on disk, another run
    d = _copy(ck, tmp_path / "w" / "checkpoints" / "step_000000003")
    a, b = (d / "batch_hasher.rank_0.bin").read_bytes(), (d / "batch_hasher.rank_1.bin").read_bytes()
    (d / "batch_hasher.rank_0.bin").write_bytes(b), (d / "batch_hasher.rank_1.bin").write_bytes(a)
    assert a != b and verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])["verified"] is False


def test_batch_chains_every_rank_is_needed_and_boundaries_cannot_move(handoff, tmp_path):
    tmp, res, ck, hashes = handoff
    d = _copy(ck, tmp_path / "m" / "checkpoints" / "step_000000003")
    whole = read_batch_digest(d, 2)
    assert len(whole) == 32 and whole != (d / "batch_hasher.rank_0.bin").read_bytes()      # rank 0 alone does not stand for the run
    assert read_batch_digest(d, 1) == (d / "batch_hasher.rank_0.bin").read_bytes()           # one rank: its chain, as the run combined it
    (d / "batch_hasher.rank_1.bin").write_bytes((d / "batch_hasher.rank_1.bin").read_bytes()[:16])
    with pytest.raises(HandoffError, match="holds 16 bytes, a chain is 32"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])
    (d / "batch_hasher.rank_1.bin").unlink()
    with pytest.raises(HandoffError, match=r"batch_hasher.rank_1.bin is missing; with dp_world_size=2"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])


def test_gradient_files_that_do_not_account_for_the_model_are_refused(handoff, tmp_path):
    from safetensors.torch import load_file, save_file

    tmp, res, ck, hashes = handoff
    ok = {"format": "pretrain-audit-gradients", "format_version": "1", "none_grad_names": "[]"}
    d = _copy(ck, tmp_path / "s" / "checkpoints" / "step_000000003")
    side = d / "gradients.safetensors"
    tensors = load_file(str(side))
    name = sorted(tensors)[0]

    def refused(match):
        with pytest.raises(HandoffError, match=match):
            verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])

    side.unlink()
    refused("is missing.*not the same as a model whose gradients were all None")
    for md in ({"format": "something-else", "format_version": "1", "none_grad_names": "[]"}, {"format": "pretrain-audit-gradients", "format_version": "2", "none_grad_names": "[]"}):
        save_file(tensors, str(side), metadata=md)
        refused("format tag")
    save_file(tensors, str(side), metadata={"format": "pretrain-audit-gradients", "format_version": "1"})
    refused(r"does not parse as a gradient file \(KeyError")
    for bad in ('{"a": 1}', "[1, 2]", "not json"):
        save_file(tensors, str(side), metadata=dict(ok, none_grad_names=bad))
        refused("none_grad_names is not a list of names|does not parse as a gradient file")
    side.write_bytes(b"\x00" * 64)
    refused("does not parse as a gradient file")
    save_file(tensors, str(side), metadata=dict(ok, none_grad_names=json.dumps([name])))
    refused("has a tensor AND is listed as having no gradient")
    save_file(tensors, str(side), metadata=dict(ok, none_grad_names=json.dumps(["x.y", "x.y"])))
    refused("a name appears twice in none_grad_names")
    save_file(dict(tensors, **{"not.a.parameter": torch.zeros(2)}), str(side), metadata=ok)
    refused("names parameters the model does not have: not.a.parameter")
    fewer = dict(tensors)
    fewer.pop(name)
    save_file(fewer, str(side), metadata=ok)
    refused("says nothing about %s" % name.replace(".", r"\."))
    save_file(dict(fewer, **{name: tensors[name].reshape(-1)[:-1].clone()}), str(side), metadata=ok)    # another model's shape
    refused("%s comes as torch.float32" % name.replace(".", r"\."))
    save_file(dict(fewer, **{name: tensors[name].to(torch.bfloat16)}), str(side), metadata=ok)
    refused("comes as torch.bfloat16")
    # an explicit zero gradient is not an absent one: naming the parameter in none_grad_names instead is accepted by the
    # reader but hashes as this engine hashes a zero gradient, so only a tensor that really was zero would still verify
    save_file(fewer, str(side), metadata=dict(ok, none_grad_names=json.dumps([name])))
    assert verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])["verified"] is False


def test_a_training_checkpoint_without_gradients_is_not_a_hand_off(handoff):
    tmp, res, ck, hashes = handoff
    with pytest.raises(HandoffError, match="gradients.safetensors is missing"):
        verify_handoff(res["run_dir"] + "/checkpoints/step_000000002", expect_hash=hashes[2], prev_hash=hashes[1])


def test_incomplete_self_contradicting_and_off_cadence_artifacts_are_refused(handoff, tmp_path):
    tmp, res, ck, hashes = handoff
    kw = dict(expect_hash=hashes[3], prev_hash=hashes[2])
    d = _copy(ck, tmp_path / "c" / "checkpoints" / "step_000000003")
    (d / "_COMPLETE").unlink()
    with pytest.raises(HandoffError, match="has no _COMPLETE marker"):
        verify_handoff(str(d), **kw)
    d = _copy(ck, tmp_path / "n" / "checkpoints" / "step_000000003")
    (d / "meta.json").unlink()
    with pytest.raises(HandoffError, match="meta.json is missing, so neither topology nor hash cadence"):
        verify_handoff(str(d), **kw)
    (d / "meta.json").write_text("[1, 2")
    with pytest.raises(HandoffError, match="is not readable JSON"):
        verify_handoff(str(d), **kw)
    (d / "meta.json").write_text("[1, 2]")
    with pytest.raises(HandoffError, match="expected a JSON object"):
        verify_handoff(str(d), **kw)
    for step in (None, 0, -3, "3", 3.0, True):
        d2 = _copy(ck, tmp_path / ("st%r" % (step,)).replace(".", "_") / "checkpoints" / "step_000000003")
        _edit_meta(d2, step=step)
        with pytest.raises(HandoffError, match="step has to be a positive integer"):
            verify_handoff(str(d2), **kw)
    # the artifact's own claim disagrees with the published value: refused before anything is loaded
    d = _copy(ck, tmp_path / "claim" / "checkpoints" / "step_000000003")
    with pytest.raises(HandoffError, match="the directory and the published log disagree about step 3"):
        verify_handoff(str(d), expect_hash="5" * 64, prev_hash=hashes[2])
    # state_hash.txt that is not the running chain (an off-cadence side link, or a doctored file)
    (d / "state_hash.txt").write_text("7" * 64 + "\n")
    with pytest.raises(HandoffError, match="is not the running chain recorded in meta.json"):
        verify_handoff(str(d), **kw)
    # a cadence the step is not on, and a run that never hashed
    d = _copy(ck, tmp_path / "cad" / "checkpoints" / "step_000000003")
    cfg = json.loads(json.loads((d / "meta.json").read_text())["config_resolved"])
    cfg["train"]["state_hash"]["every_n_steps"] = 2
    _edit_meta(d, config_resolved=json.dumps(cfg))
    with pytest.raises(HandoffError, match="lies between hashed steps"):
        verify_handoff(str(d), **kw)
    cfg["train"]["state_hash"]["every_n_steps"] = 0
    _edit_meta(d, config_resolved=json.dumps(cfg))
    with pytest.raises(HandoffError, match="never hashed its state"):
        verify_handoff(str(d), **kw)


@pytest.mark.parametrize("bad", [dict(dp_world_size=10 ** 6, dp_shard=10 ** 6), dict(dp_world_size=2, dp_replicate=-1, dp_shard=-2),
                                 dict(dp_world_size=4, dp_replicate=1, dp_shard=2), dict(dp_world_size="2")])
def test_an_implausible_topology_is_refused(handoff, tmp_path, bad):
    tmp, res, ck, hashes = handoff
    d = _copy(ck, tmp_path / "checkpoints" / "step_000000003")
    _edit_meta(d, **bad)
    with pytest.raises(HandoffError, match="is implausible|does not multiply out"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])


def test_the_wrong_topology_fails_the_comparison(handoff, tmp_path):
    """a plausible but untrue topology is not refused - it is an input of the digest and simply does not reproduce it"""
    tmp, res, ck, hashes = handoff
    d = _copy(ck, tmp_path / "checkpoints" / "step_000000003")
    _edit_meta(d, dp_world_size=2, dp_replicate=2, dp_shard=1)
    assert verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])["verified"] is False


def test_cheap_refusals_do_not_apply_the_checkpoints_environment(handoff, tmp_path, monkeypatch):
    tmp, res, ck, hashes = handoff
    d = _copy(ck, tmp_path / "checkpoints" / "step_000000003")
    _edit_meta(d, kernel_env={"OTB_GEMM_PLAIN_TEST_MARK": "1", "PRETRAIN_AUDIT_STREAM_HEAD": "1"}, dp_world_size=10 ** 6)
    before = dict(os.environ)
    with pytest.raises(HandoffError, match="is implausible"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])
    assert dict(os.environ) == before
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    d = _copy(ck, tmp_path / "dev" / "checkpoints" / "step_000000003")
    with pytest.raises(HandoffError, match="no CUDA device here"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2], device="cuda")
    with pytest.raises(HandoffError, match="can be held on cpu or cuda"):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2], device="meta")
    # metadata that tries to redirect native code is refused as a hand-off error, not applied
    _edit_meta(d, kernel_env={"LD_PRELOAD": "/tmp/x.so"})
    with pytest.raises(HandoffError):
        verify_handoff(str(d), expect_hash=hashes[3], prev_hash=hashes[2])
    assert "LD_PRELOAD" not in os.environ or os.environ["LD_PRELOAD"] == before.get("LD_PRELOAD")


def test_command_line_round_trip_tampering_and_json_result(handoff, tmp_path, capsys, monkeypatch):
    tmp, res, ck, hashes = handoff
    out = tmp_path / "result.json"
    assert verify_main(["--checkpoint", ck, "--expect-hash", hashes[3], "--prev-hash", hashes[2], "--json", str(out)]) == 0
    printed = json.loads(capsys.readouterr().out)
    assert printed["verified"] is True and json.loads(out.read_text()) == printed
    # a mismatch: exit status 1, both digests in full on the error stream, and the result file replaced
    assert verify_main(["--checkpoint", ck, "--expect-hash", hashes[3], "--prev-hash", hashes[1], "--json", str(out)]) == 1
    io = capsys.readouterr()
    assert json.loads(io.out)["verified"] is False and json.loads(out.read_text())["verified"] is False
    assert "AUDIT FAILED: state_hash" in io.err and hashes[3] in io.err
    # a refusal overwrites an earlier success instead of leaving it to be read as this run's answer
    out.write_text(json.dumps({"verified": True}))
    assert verify_main(["--checkpoint", ck, "--expect-hash", "abc", "--prev-hash", hashes[2], "--json", str(out)]) == 1
    refusal = json.loads(out.read_text())
    assert refusal["verified"] is False and "--expect-hash takes the 64 hex digits" in refusal["error"]
    capsys.readouterr()
    # an unexpected failure (here: the tensor payload is gone) is reported with its type, as JSON, not as a traceback exit
    d = _copy(ck, tmp_path / "broken" / "checkpoints" / "step_000000003")
    shutil.rmtree(d / "dcp")
    assert verify_main(["--checkpoint", str(d), "--expect-hash", hashes[3], "--prev-hash", hashes[2], "--json", str(out)]) == 1
    broken = json.loads(capsys.readouterr().out)
    assert broken["verified"] is False and ":" in broken["error"] and json.loads(out.read_text()) == broken
    # a result file that cannot be written fails closed
    assert verify_main(["--checkpoint", ck, "--expect-hash", hashes[3], "--prev-hash", hashes[2], "--json", str(tmp_path / "no_dir" / "r.json")]) == 1
    assert "cannot write" in json.loads(capsys.readouterr().out)["error"]
    # both commitments are required
    for missing in (["--expect-hash", hashes[3]], ["--prev-hash", hashes[2]]):
        with pytest.raises(SystemExit):
            verify_main(["--checkpoint", ck, *missing])
    capsys.readouterr()


def test_verify_loaded_state_clears_the_gradients_it_attached(handoff):
    from open_transformers_b200.config import parse_config_resolved
    from open_transformers_b200.train.checkpoint import Checkpointer
    from open_transformers_b200.train.engine import TrainEngine

    tmp, res, ck, hashes = handoff
    meta = Checkpointer.read_meta(ck)
    cfg = parse_config_resolved(meta.config_resolved)
    cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size = meta.dp_world_size, meta.dp_shard, meta.dp_replicate
    engine = TrainEngine(cfg, "cpu", 0, 1, init=False)
    Checkpointer(Path(ck).parent.parent).load(ck, engine)
    r = VH.verify_loaded_state(engine, ck, expect_hash=hashes[3], prev_hash=hashes[2], include_grads=True, include_batch=True,
                               tensor_digest=meta.tensor_digest)
    assert r["verified"] is True and r["gradients_attached"] == len(engine.names) and float(engine.grad_red.abs().sum()) == 0.0
    # without the gradient or batch term another schema is hashed: the commitment is not reproduced
    for kw in (dict(include_grads=False, include_batch=True), dict(include_grads=True, include_batch=False)):
        r = VH.verify_loaded_state(engine, ck, expect_hash=hashes[3], prev_hash=hashes[2], tensor_digest=meta.tensor_digest, **kw)
        assert r["verified"] is False and (r["gradients_attached"] is None) == (not kw["include_grads"])
    engine.close()
