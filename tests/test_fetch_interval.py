"""The interval fetcher: only the shards an interval reads come as real bytes (verified against the manifest), the rest as
sparse stand-ins; a second, longer fetch keeps what it verified and replaces the stand-ins that became touched; the walk
from the stream's origin serves ``--from-init`` replays; a token-clocked recipe gets its default span from the schedule.
(reference test strategy: tests/test_fetch_interval.py - fake mirror injected, no network)"""
import json
import shutil
from pathlib import Path

import pytest

from helpers import tiny_cfg
from open_transformers_b200.cli.audit_replay import audit_replay
from open_transformers_b200.data.fetch_interval import DirMirror, FetchIntegrityError, fetch_audit_interval
from open_transformers_b200.train.batch_schedule import default_interval_end
from open_transformers_b200.train.loop import train


class CountingMirror(DirMirror):
    def __init__(self, root):
        super().__init__(root)
        self.downloads = []

    def download(self, rel, dest):
        self.downloads.append(str(rel))
        super().download(rel, dest)


@pytest.fixture(scope="module")
def run(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("fetch"))
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=1"])
    res = train(cfg, device="cpu", data_root=tmp)
    return tmp, cfg, res


def test_fetch_result_manifest_stubs_and_resume(run, tmp_path):
    tmp, cfg, res = run
    ck = Path(res["run_dir"]) / "checkpoints" / "step_000000001"
    dest = tmp_path / "data"
    mirror = CountingMirror(tmp)
    r = fetch_audit_interval(ck, mirror, dest, until_step=2)
    assert (r.start_step, r.until_step, r.from_init, r.verified) == (1, 2, False, True) and r.data_root == str(dest)
    assert json.loads((dest / "fetch_manifest.json").read_text())["touched_shards"] == r.touched_shards
    bins = sorted(dest.rglob("*.bin"))
    real = [b for b in bins if b.stat().st_blocks > 0]
    assert r.bytes_fetched == sum(b.stat().st_size for b in real) > 0 and r.stubs_created == len(bins) - len(real)
    assert sum(len(v) for v in r.touched_shards.values()) == len(real)
    assert audit_replay(str(ck), data_root=str(dest), until_step=2, expect_hash=dict(res["hashes"])[2])["match"] is True
    # the same fetch again: nothing but manifests travels, nothing is stubbed anew
    mirror.downloads.clear()
    again = fetch_audit_interval(ck, mirror, dest, until_step=2)
    assert again.bytes_fetched == 0 and again.stubs_created == 0 and all(d.endswith("manifest.yaml") for d in mirror.downloads)
    # a longer interval: the stand-ins that became touched are replaced by real, verified bytes
    longer = fetch_audit_interval(ck, mirror, dest, until_step=3)
    newly = {(k, s) for k, v in longer.touched_shards.items() for s in v} - {(k, s) for k, v in r.touched_shards.items() for s in v}
    assert (longer.bytes_fetched > 0) == bool(newly)
    assert audit_replay(str(ck), data_root=str(dest), until_step=3, expect_hash=dict(res["hashes"])[3])["match"] is True


def test_default_span_and_the_walk_from_the_origin(run, tmp_path):
    tmp, cfg, res = run
    ck = Path(res["run_dir"]) / "checkpoints" / "step_000000002"
    r = fetch_audit_interval(ck, DirMirror(tmp), tmp_path / "d1")
    assert (r.start_step, r.until_step) == (2, 3)                       # one checkpoint interval of the recipe
    o = fetch_audit_interval(ck, DirMirror(tmp), tmp_path / "d2", from_init=True)
    assert (o.start_step, o.start_consumed_tokens, o.until_step, o.from_init) == (0, 0, 2, True)
    replay = audit_replay(str(ck), data_root=str(tmp_path / "d2"), from_init=True, until_step=2, expect_hash=dict(res["hashes"])[2])
    assert replay["match"] is True
    with pytest.raises(ValueError, match="not beyond the starting step"):
        fetch_audit_interval(ck, DirMirror(tmp), tmp_path / "d3", until_step=2)
    # a recipe that clocks checkpoints by tokens: the span ends at the first step across the next multiple
    tr = cfg.train.model_copy(update={"ckpt_every_steps": 0, "ckpt_every_tokens": 600})
    per_step = cfg.train.global_batch_tokens.warmup
    assert default_interval_end(0, 0, tr) == -(-600 // per_step) and default_interval_end(5, 5 * per_step, cfg.train) == 6


def test_a_corrupt_mirror_is_noticed_and_leaves_no_payload_behind(run, tmp_path):
    tmp, cfg, res = run
    ck = Path(res["run_dir"]) / "checkpoints" / "step_000000001"
    touched = fetch_audit_interval(ck, DirMirror(tmp), tmp_path / "ok", until_step=2).touched_shards
    bad = tmp_path / "mirror"
    for src in cfg.data.sources:
        shutil.copytree(Path(tmp) / src.path, bad / src.path)
    name, ids = next((k, v) for k, v in touched.items() if v)
    victim = next(p for src in cfg.data.sources for p in sorted((bad / src.path).glob("*.bin"))
                  if (bad / src.path / "manifest.yaml").read_text().find(name) >= 0)
    # flip one byte in every payload of that source: whichever shard the interval reads, its digest no longer matches
    for p in victim.parent.glob("*.bin"):
        raw = bytearray(p.read_bytes())
        raw[len(raw) // 2] ^= 0xFF
        p.write_bytes(bytes(raw))
    dest = tmp_path / "bad_dest"
    with pytest.raises(FetchIntegrityError, match="does not match its manifest digest"):
        fetch_audit_interval(ck, DirMirror(bad), dest, until_step=2)
    assert not [b for b in dest.rglob("*.bin") if b.parent.name == victim.parent.name and b.stat().st_blocks > 0]
    # unverified, the same mirror is accepted (and a replay on it then fails the hash, loudly)
    r = fetch_audit_interval(ck, DirMirror(bad), tmp_path / "unverified", until_step=2, verify=False)
    assert r.verified is False and r.bytes_fetched > 0
    with pytest.raises(FileNotFoundError, match="mirror lacks"):
        fetch_audit_interval(ck, DirMirror(tmp_path / "nothing"), tmp_path / "none", until_step=2)
