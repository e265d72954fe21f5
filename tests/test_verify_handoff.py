"""Hand-off verification from disk alone: a checkpoint saved by the replay carries its post-clip gradients; the verifier
rebuilds the chained hash without a forward or backward pass and notices any altered tensor, gradient, batch digest or
previous link. (reference test strategy: tests/test_verify_handoff.py, tests/test_audit_gradient_sidecar.py)"""
import json
import shutil
from pathlib import Path

import pytest
import torch

from helpers import tiny_cfg
from open_transformers_b200.cli.audit_replay import audit_replay
from open_transformers_b200.cli.verify_handoff import (main as verify_main, read_gradient_sidecar, verify_handoff,
                                                       write_gradient_sidecar)
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


def test_verifier_accepts_the_saved_checkpoint_and_needs_the_right_previous_link(handoff, capsys):
    tmp, res, ck, hashes = handoff
    v = verify_handoff(ck, prev_hash=hashes[2])
    assert v["match"] is True and v["state_hash"] == hashes[3] and v["step"] == 3
    assert verify_handoff(ck, expect_hash=hashes[3], prev_hash=hashes[2])["match"] is True
    assert verify_handoff(ck, prev_hash=hashes[1])["match"] is False
    assert verify_main(["--checkpoint", ck, "--prev-hash", hashes[2]]) == 0
    assert "MATCH=True" in capsys.readouterr().out
    assert verify_main(["--checkpoint", ck, "--prev-hash", hashes[2], "--expect-hash", "0" * 64, "--json"]) == 1
    io = capsys.readouterr()
    assert json.loads(io.out)["match"] is False and "AUDIT FAILED: state_hash" in io.err


def test_sidecar_round_trip_keeps_absent_gradients_apart_from_zero_ones(tmp_path):
    g = {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "b": None, "c": torch.zeros(4)}
    write_gradient_sidecar(tmp_path, g)
    back = read_gradient_sidecar(tmp_path)
    assert set(back) == {"a", "b", "c"} and back["b"] is None and torch.equal(back["a"], g["a"]) and torch.equal(back["c"], g["c"])


def test_any_altered_input_is_noticed(handoff, tmp_path):
    from safetensors.torch import load_file, save_file

    tmp, res, ck, hashes = handoff
    # one gradient element, one unit in the last place
    d = _copy(ck, tmp_path / "g" / "checkpoints" / "step_000000003")
    grads = read_gradient_sidecar(d)
    name = sorted(n for n, t in grads.items() if t is not None and t.numel() > 10)[0]
    grads[name].view(-1).view(torch.int32)[3] ^= 1
    write_gradient_sidecar(d, grads)
    assert verify_handoff(str(d), prev_hash=hashes[2])["match"] is False
    # a batch digest
    d = _copy(ck, tmp_path / "b" / "checkpoints" / "step_000000003")
    raw = bytearray((d / "batch_hasher.rank_1.bin").read_bytes())
    raw[31] ^= 0x80
    (d / "batch_hasher.rank_1.bin").write_bytes(bytes(raw))
    assert verify_handoff(str(d), prev_hash=hashes[2])["match"] is False
    (d / "batch_hasher.rank_1.bin").write_bytes(bytes(raw[:16]))
    with pytest.raises(ValueError):
        verify_handoff(str(d), prev_hash=hashes[2])
    # no sidecar, a foreign sidecar, a sidecar without one of the parameters
    d = _copy(ck, tmp_path / "s" / "checkpoints" / "step_000000003")
    side = d / "gradients.safetensors"
    tensors = load_file(str(side))
    side.unlink()
    with pytest.raises(FileNotFoundError):
        verify_handoff(str(d), prev_hash=hashes[2])
    save_file(tensors, str(side), metadata={"format": "something-else", "format_version": "1"})
    with pytest.raises(ValueError):
        verify_handoff(str(d), prev_hash=hashes[2])
    tensors.pop(name)
    save_file(tensors, str(side), metadata={"format": "pretrain-audit-gradients", "format_version": "1", "none_grad_names": "[]"})
    with pytest.raises(KeyError):
        verify_handoff(str(d), prev_hash=hashes[2])


def test_a_training_checkpoint_without_gradients_is_not_a_hand_off(handoff):
    tmp, res, ck, hashes = handoff
    with pytest.raises(FileNotFoundError):
        verify_handoff(res["run_dir"] + "/checkpoints/step_000000002", prev_hash=hashes[1])
