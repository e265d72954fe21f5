"""The replay's preflight: everything that can be refused from the command line and ``meta.json`` alone is refused before a
model is built or a checkpoint payload is read. ``meta.json`` is untrusted input.
(reference test strategy: tests/test_audit_meta_bounds.py, test_audit_device_guard.py, test_audit_until_step_guard.py,
test_audit_expect_hash.py, test_audit_mismatch_message.py, test_audit_kit_provenance.py, test_checkpoint_cold_start_guard.py)"""
import json
import re

import pytest
import torch

from open_transformers_b200.cli import audit_replay as AR
from open_transformers_b200.config import load_config
from open_transformers_b200.train.checkpoint import resolved_config_json

SHAPE = ["model.n_layers=1", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2", "model.ffn_intermediate=256", "model.vocab_size=256"]


def meta_only_checkpoint(tmp_path, **over):
    """A checkpoint directory that holds nothing but meta.json: a guard that lets it through fails later, on the missing
    payload, with another error type."""
    cfg = load_config("tiny_cpu", SHAPE)
    d = tmp_path / "runs" / "t" / "checkpoints" / "step_000000010"
    d.mkdir(parents=True)
    meta = {"seed": cfg.run.seed, "step": 10, "consumed_tokens": 10 * 1024, "chained_hash": "ab" * 32, "reduction_mode": "deterministic_allgather",
            "dp_world_size": 2, "dp_replicate": 1, "dp_shard": 2, "config_resolved": resolved_config_json(cfg), "repop_env": {}}
    meta.update(over)
    (d / "meta.json").write_text(json.dumps(meta))
    return str(d)


@pytest.mark.parametrize("over,what", [
    (dict(dp_world_size=10 ** 6, dp_shard=10 ** 6), "out of bounds"),
    (dict(dp_world_size=AR.MAX_AUDIT_WORLD + 1, dp_shard=AR.MAX_AUDIT_WORLD + 1), "out of bounds"),
    (dict(dp_world_size=2, dp_replicate=-1, dp_shard=-2), "out of bounds"),          # the product alone would pass
    (dict(dp_world_size=4, dp_replicate=1, dp_shard=2), "out of bounds"),
    (dict(dp_world_size=0, dp_replicate=0, dp_shard=1), "out of bounds"),
    (dict(step=-1), "negative"),
    (dict(consumed_tokens=-5), "negative"),
    (dict(replicate_reduce_algo="ascending_allgather"), "replica orders"),
    (dict(replicate_reduce_algo="binary_blocks_tree", dp_world_size=7, dp_replicate=7, dp_shard=1), "replica orders"),   # the earlier stride tree differs at 7
    (dict(clip_algo="per_tensor"), "clip / norm"),
])
def test_implausible_metadata_is_refused_before_anything_is_built(tmp_path, over, what):
    ck = meta_only_checkpoint(tmp_path, **over)
    with pytest.raises(AR.AuditError, match=what):
        AR.audit_replay(ck, device="cpu")


def test_plausible_metadata_passes_the_gate_and_fails_later_on_the_missing_payload(tmp_path):
    for i, over in enumerate([dict(dp_world_size=8, dp_replicate=2, dp_shard=4), dict(replicate_reduce_algo="recursive_doubling"),
                              dict(replicate_reduce_algo="binary_blocks_tree", dp_world_size=6, dp_replicate=6, dp_shard=1)]):
        ck = meta_only_checkpoint(tmp_path / str(i), **over)
        with pytest.raises(Exception) as e:
            AR.audit_replay(ck, device="cpu", until_step=11)
        assert not isinstance(e.value, AR.AuditError), over


@pytest.mark.parametrize("until_step", [10, 9, 0, -3])
def test_until_step_at_or_below_the_start_is_refused_early(tmp_path, until_step):
    ck = meta_only_checkpoint(tmp_path)
    with pytest.raises(AR.AuditError, match="not beyond the starting step 10"):
        AR.audit_replay(ck, device="cpu", until_step=until_step)


def test_device_guard(tmp_path, monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    for dev in ("cuda", "cuda:0", "cuda:3"):
        with pytest.raises(AR.AuditError, match="no CUDA device is visible"):
            AR.check_device(dev)
    for dev in ("mps", "mps:0", "xpu", "cuda:x"):
        with pytest.raises(AR.AuditError, match="cpu or cuda"):
            AR.check_device(dev)
    AR.check_device("cpu")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 2)
    AR.check_device("cuda:1")
    with pytest.raises(AR.AuditError, match="only 2 CUDA device"):
        AR.check_device("cuda:2")
    # the guard runs inside the replay, ahead of the metadata
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(AR.AuditError, match="no CUDA device"):
        AR.audit_replay(meta_only_checkpoint(tmp_path), device="cuda")


def test_a_gpu_replay_on_an_installation_without_kernels_names_the_missing_library(tmp_path, monkeypatch):
    from open_transformers_b200 import build_native

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)
    monkeypatch.setattr(build_native, "EXT", tmp_path / "no_ext")

    def no_compiler():
        raise RuntimeError("nvcc not found")

    monkeypatch.setattr(build_native, "_nvcc", no_compiler)
    with pytest.raises(AR.AuditError, match="libotb_cuda.so is missing"):
        AR.check_device("cuda")
    AR.check_device("cpu")   # the CPU replay needs no GPU build


def test_expect_hash_forms(tmp_path, monkeypatch):
    d = "AB" * 32
    assert AR.resolve_expect_hash(d) == d.lower() and AR.resolve_expect_hash("  %s\n" % d) == d.lower() and AR.resolve_expect_hash(None) is None
    for n in (8, 16, 63, 65):
        with pytest.raises(AR.AuditError, match="64-character hex digest"):
            AR.resolve_expect_hash("a" * n)
    with pytest.raises(AR.AuditError):
        AR.resolve_expect_hash(str(tmp_path / "missing.txt"))
    f = tmp_path / "hash.txt"
    f.write_text(d + "  step_000000010\n")
    assert AR.resolve_expect_hash(str(f)) == d.lower()
    f.write_text("not a digest\n")
    with pytest.raises(AR.AuditError, match="does not start with a 64-hex digest"):
        AR.resolve_expect_hash(str(f))
    f.write_text("abcdef12\n")
    with pytest.raises(AR.AuditError):
        AR.resolve_expect_hash(str(f))
    assert len(d) == 2 * 32   # the digest length is that of the state hash (blake2b-256)


def test_mismatch_message_carries_both_digests_in_full():
    got, want = "1a" * 32, "2b" * 32
    msg = AR.mismatch_message(got, want)
    assert got in msg and want in msg and "..." not in msg
    assert re.findall(r"[0-9a-f]{64}", msg) == [got, want]   # what a log parser recovers


def test_cold_start_guard_refuses_a_run_directory_that_already_holds_checkpoints(tmp_path):
    from helpers import tiny_cfg
    from open_transformers_b200.train.loop import train

    cfg = tiny_cfg(str(tmp_path), ["train.ckpt_every_steps=2", "train.total_tokens=512"])
    res = train(cfg, device="cpu", data_root=str(tmp_path))
    with pytest.raises(RuntimeError, match="already holds checkpoints"):
        train(cfg, device="cpu", data_root=str(tmp_path))
    # unrelated files do not count, and a resume is not a cold start
    other = tiny_cfg(str(tmp_path), ["train.ckpt_every_steps=2", "train.total_tokens=512", "run.run_id=fresh"])
    (tmp_path / "runs" / "fresh" / "checkpoints").mkdir(parents=True)
    (tmp_path / "runs" / "fresh" / "checkpoints" / "notes.txt").write_text("x")
    assert train(other, device="cpu", data_root=str(tmp_path))["step"] == res["step"]
