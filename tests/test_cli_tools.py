"""The data-preparation and checkpoint command-line tools, end to end on small inputs: tokenizer training, sharding
(whole files and a byte segment), manifest merge, shard inspection, token statistics, synthetic sources, the windows of a
step, document dump to Parquet, checkpoint inspection and fingerprint.
(reference: src/pretrain/cli/prepare_data.py:300-378, cli/dump_documents.py, cli/inspect_checkpoint.py, cli/hash_ckpt.py)"""
import json
import shutil
from pathlib import Path

import pytest

from helpers import tiny_cfg

tokenizers = pytest.importorskip("tokenizers")


def _run(main, argv, capsys):
    capsys.readouterr()
    rc = main(argv)
    return rc, capsys.readouterr().out


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    root = tmp_path_factory.mktemp("corpus")
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "12", "345", "6789"]
    paths = []
    for f in range(2):
        p = root / ("part%d.jsonl" % f)
        with open(p, "w") as fh:
            for i in range(60):
                fh.write(json.dumps({"text": " ".join(words[(i * 7 + j * 3 + f) % len(words)] for j in range(5 + i % 9)), "id": i}) + "\n")
        paths.append(str(p))
    return root, paths


def test_tokenizer_shards_manifests_and_dumps(corpus, capsys):
    from open_transformers_b200.cli.dump_documents import main as dump_main
    from open_transformers_b200.cli.prepare_data import main as prep
    from open_transformers_b200.data.indexed_dataset import IndexedDatasetReader
    from open_transformers_b200.data.manifest import SourceManifest
    from open_transformers_b200.data.tokenizer import Tokenizer, compute_hash

    root, paths = corpus
    tok_path = str(root / "tok.json")
    rc, out = _run(prep, ["train-tokenizer", *paths, "--output", tok_path, "--vocab-size", "320", "--min-frequency", "1"], capsys)
    assert rc == 0 and json.loads(out)["hash"] == compute_hash(tok_path)
    tok = Tokenizer(tok_path)
    assert tok.decode(tok.encode("alpha 345 kappa")) == "alpha 345 kappa" and tok.eos_id is not None

    rc, out = _run(prep, ["shard", *paths, "--tokenizer", tok_path, "--out-dir", str(root / "src_a"), "--name", "a", "--shard-bytes", "1024"], capsys)
    info = json.loads(out)
    assert rc == 0 and info["documents"] == 120 and info["shards"] >= 2
    man = SourceManifest.load(root / "src_a" / "manifest.yaml")
    assert man.total_documents == 120 and man.verify(root / "src_a") == [] and man.tokenizer_hash == compute_hash(tok_path)
    first = IndexedDatasetReader(root / "src_a" / man.shards[0].prefix)
    assert tok.decode(first.document(0)) == json.loads(open(paths[0]).readline())["text"]

    # a byte segment of one file (what the fan-out workers do): the two halves together hold every document of the file
    size = (root / "part0.jsonl").stat().st_size
    docs = 0
    for k, (lo, hi) in enumerate(((0, size // 2), (size // 2, size))):
        rc, out = _run(prep, ["shard", paths[0], "--tokenizer", tok_path, "--out-dir", str(root / ("seg%d" % k)), "--name", "seg%d" % k,
                              "--segment", "%d:%d" % (lo, hi)], capsys)
        docs += json.loads(out)["documents"]
    assert docs == 60
    rc, out = _run(prep, ["merge-manifests", str(root / "seg0" / "manifest.yaml"), str(root / "seg1" / "manifest.yaml"), "--name", "merged",
                          "--output", str(root / "merged.yaml")], capsys)
    assert rc == 0 and SourceManifest.load(root / "merged.yaml").total_documents == 60

    rc, out = _run(prep, ["token-stats", str(root / "src_a" / "manifest.yaml"), str(root / "merged.yaml")], capsys)
    rows = json.loads(out)
    assert [r["name"] for r in rows] == ["a", "merged"] and abs(sum(r["token_share"] for r in rows) - 1) < 1e-9
    rc, out = _run(prep, ["inspect", str(root / "src_a" / man.shards[0].prefix), "--tokenizer", tok_path, "--docs", "2"], capsys)
    assert rc == 0 and "alpha" in out or "beta" in out

    # the documents table: one file per shard under <out>/<source>/, keyed like the step -> document map; a second run skips
    rc, out = _run(dump_main, ["--data-root", str(root), "--tokenizer", tok_path, "--out-dir", str(root / "dump"), "--workers", "1", "--batch-docs", "50"], capsys)
    import pyarrow.parquet as pq

    files = sorted((root / "dump").rglob("*.parquet"))
    assert rc == 0 and files and not list((root / "dump").rglob("*.part"))
    first_file = root / "dump" / man.name / ("00000_%s.parquet" % Path(man.shards[0].prefix).name)
    table = pq.read_table(first_file).to_pylist()
    assert list(table[0]) == ["source", "shard_id", "local_doc", "n_tokens", "text"]
    assert table[0]["text"] == json.loads(open(paths[0]).readline())["text"] and table[0]["n_tokens"] == first.document_length(0)
    assert table[0]["source"] == man.name and table[0]["shard_id"] == 0 and [r["local_doc"] for r in table] == list(range(len(table)))
    assert sum(len(pq.read_table(f)) for f in files if f.parent.name == man.name) == 120
    stamp = first_file.stat().st_mtime_ns
    rc, _ = _run(dump_main, ["--data-root", str(root), "--tokenizer", tok_path, "--out-dir", str(root / "dump"), "--workers", "1", "--sources", man.name,
                             "--limit-shards", "1"], capsys)
    assert rc == 0 and first_file.stat().st_mtime_ns == stamp
    assert dump_main(["--data-root", str(root / "nothing_here"), "--tokenizer", tok_path, "--out-dir", str(root / "dump2"), "--workers", "1"]) == 1


def test_synthetic_sources_step_windows_and_checkpoint_tools(tmp_path, capsys):
    from open_transformers_b200.cli.hash_ckpt import hash_checkpoint, main as hash_main
    from open_transformers_b200.cli.inspect_checkpoint import main as inspect_main
    from open_transformers_b200.cli.prepare_data import main as prep
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=2"])
    over = ["train.seq_len=64", "data.seq_len=64", "model.max_seq_len_pretrain=64", "train.micro_batch_size=2",
            "train.global_batch_tokens.warmup=256", "train.global_batch_tokens.main=256", "train.global_batch_tokens.late=256"]
    rc, out = _run(prep, ["replay-step", "--config-name", "tiny_cpu", "--data-root", tmp, "--step", "1", "--max-tokens", "8", *over], capsys)
    rows = [json.loads(l) for l in out.splitlines()]
    assert rc == 0 and len(rows) == 4 and all(r["step"] == 1 and len(r["tokens"]) == 8 for r in rows)
    assert sorted((r["dp_rank"], r["slot"]) for r in rows) == [(0, 0), (0, 1), (1, 0), (1, 1)]

    res = train(cfg, device="cpu", data_root=tmp)
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    rc, out = _run(inspect_main, [ck], capsys)
    assert rc == 0 and '"step": 2' in out and "complete: True" in out and dict(res["hashes"])[2] in out and "bytes, --full-config" in out
    rc, out = _run(hash_main, [ck], capsys)
    assert rc == 0 and out.strip() == hash_checkpoint(ck) and len(out.strip()) == 64
    rc, weights_only = _run(hash_main, [ck, "--weights-only"], capsys)
    assert weights_only.strip() != out.strip()
    # --config-name checks the checkpoint against that recipe's model: the run's own shape passes, the stock one does not
    shape = ["model.n_layers=1", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2", "model.ffn_intermediate=256", "model.vocab_size=256"]
    rc, again = _run(hash_main, [ck, "--config-name", "tiny_cpu", "--override", *shape], capsys)
    assert rc == 0 and again.strip() == out.strip()
    with pytest.raises(ValueError, match="does not match configuration tiny_cpu"):
        hash_main([ck, "--config-name", "tiny_cpu"])
    assert hash_checkpoint(res["run_dir"] + "/checkpoints/step_000000003") != hash_checkpoint(ck)
    rc, out = _run(inspect_main, [ck, "--full-config"], capsys)
    assert rc == 0 and "bytes, --full-config" not in out and "vocab_size" in out
    from open_transformers_b200.cli.dcp_safetensors import main as st_main

    rc, out = _run(st_main, ["pack", ck, str(tmp_path / "one.safetensors")], capsys)
    assert rc == 0 and json.loads(out)["tensors"] > 0
    rc, out = _run(st_main, ["unpack", str(tmp_path / "one.safetensors"), str(tmp_path / "un" / "checkpoints" / "step_000000002")], capsys)
    assert rc == 0 and hash_checkpoint(json.loads(out)["dir"]) == hash_checkpoint(ck)

    # the reference's command names and switches: to-safetensors / from-safetensors, --verify, --keys, --top-level-key
    import torch
    from safetensors import safe_open
    from safetensors.torch import save_file

    from open_transformers_b200.cli import dcp_safetensors as DS

    full = tmp_path / "full.safetensors"
    rc, out = _run(st_main, ["to-safetensors", ck, str(full), "--verify"], capsys)
    info = json.loads(out)
    assert rc == 0 and info["verified"] and info["top_level_keys"] == ["model", "optim"] and "meta.json" in info["sidecar_files"]
    with safe_open(str(full), framework="pt") as f:
        header = f.metadata()
        names = set(f.keys())
    assert header["pretrain.format"] == "dcp-safetensors/1" and "pretrain.skeleton" in header and "pretrain.sidecar" in header
    assert "optim.state.0.exp_avg" in names and any(n.startswith("__sidecar__.rng.") for n in names)
    back = tmp_path / "back" / "checkpoints" / "step_000000002"
    rc, out = _run(st_main, ["from-safetensors", str(full), str(back), "--verify"], capsys)
    assert rc == 0 and json.loads(out)["verified"] and (back / "_COMPLETE").exists() and (back / "dcp" / ".metadata").exists()
    for name in ("meta.json", "state_hash.txt", "global_stream.json", "spike_protocol.json", "batch_hasher.rank_1.bin"):
        assert (back / name).read_bytes() == (Path(ck) / name).read_bytes(), name
    assert DS.same_state(DS.read_dcp(back / "dcp"), DS.read_dcp(Path(ck) / "dcp"))
    assert st_main(["from-safetensors", str(full), str(back)]) == 2    # a DCP writer adds files: a non-empty target is refused
    # weights only: no sidecar travels, the way back is a bare DCP directory
    rc, out = _run(st_main, ["to-safetensors", ck, str(tmp_path / "w.safetensors"), "--keys", "model"], capsys)
    assert rc == 0 and json.loads(out)["sidecar_files"] is None and json.loads(out)["top_level_keys"] == ["model"]
    rc, out = _run(st_main, ["from-safetensors", str(tmp_path / "w.safetensors"), str(tmp_path / "bare"), "--verify"], capsys)
    assert rc == 0 and (tmp_path / "bare" / ".metadata").exists() and not (tmp_path / "bare" / "_COMPLETE").exists()
    assert st_main(["to-safetensors", ck, str(tmp_path / "x.safetensors"), "--keys", "nothing_like_this"]) == 2
    # a foreign file (no skeleton) nested under --top-level-key; NaN payloads compare equal bit for bit
    foreign = {"a.weight": torch.tensor([1.0, float("nan"), -0.0]), "b.weight": torch.arange(6, dtype=torch.int32).view(2, 3)}
    save_file(foreign, str(tmp_path / "foreign.safetensors"))
    rc, out = _run(st_main, ["from-safetensors", str(tmp_path / "foreign.safetensors"), str(tmp_path / "fdcp"), "--top-level-key", "model", "--verify"], capsys)
    assert rc == 0 and DS.same_state(DS.read_dcp(tmp_path / "fdcp"), {"model": foreign})
    assert not DS.same_bits(torch.tensor([0.0]), torch.tensor([-0.0])) and DS.same_bits(torch.tensor([float("nan")]), torch.tensor([float("nan")]))
    # names in a sidecar become paths: anything outside the allow-list is refused before a byte is written
    with safe_open(str(full), framework="pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    evil = dict(header)
    evil["pretrain.sidecar"] = header["pretrain.sidecar"].replace("meta.json", "../../escape.json")
    save_file(tensors, str(tmp_path / "evil.safetensors"), metadata=evil)
    assert st_main(["from-safetensors", str(tmp_path / "evil.safetensors"), str(tmp_path / "evil_out")]) == 2
    assert not (tmp_path / "escape.json").exists() and not (tmp_path / "evil_out" / "meta.json").exists()


def test_train_command_creates_synthetic_data_resumes_and_refuses_to_overwrite(tmp_path, capsys):
    """the console entry of training, as a subprocess user would call it: first run with --synthetic-data and --max-steps,
    then --resume-from, and a second cold start into the same run directory is refused"""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parent.parent)
    tmp = str(tmp_path)
    over = ["run.output_dir=%s/runs" % tmp, "run.run_id=cli", "model.n_layers=1", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2",
            "model.ffn_intermediate=256", "model.vocab_size=256", "train.seq_len=64", "data.seq_len=64", "model.max_seq_len_pretrain=64",
            "train.micro_batch_size=2", "train.global_batch_tokens.warmup=256", "train.global_batch_tokens.main=256",
            "train.global_batch_tokens.late=256", "train.total_tokens=1024", "train.ckpt_every_steps=2"]
    base = [sys.executable, "-m", "open_transformers_b200.cli.train", "--config-name", "tiny_cpu", "--device", "cpu", "--data-root", tmp]
    env = dict(os.environ, PYTHONPATH=root, OMP_NUM_THREADS="2", WANDB_MODE="disabled")
    first = subprocess.run(base + ["--synthetic-data", "--max-steps", "2", *over], env=env, capture_output=True, text=True, timeout=300)
    assert first.returncode == 0, first.stderr[-3000:]
    out1 = json.loads(first.stdout.strip().splitlines()[-1])
    assert out1["step"] == 2 and len(out1["hashes"]) == 2
    again = subprocess.run(base + over, env=env, capture_output=True, text=True, timeout=300)
    assert again.returncode != 0 and "cold-start overwrite guard" in again.stderr
    ck = "%s/runs/cli/checkpoints/step_000000002" % tmp
    second = subprocess.run(base + ["--resume-from", ck, *over], env=env, capture_output=True, text=True, timeout=300)
    assert second.returncode == 0, second.stderr[-3000:]
    out2 = json.loads(second.stdout.strip().splitlines()[-1])
    assert out2["step"] == 4 and [s for s, _ in out2["hashes"]] == [3, 4]
    rows = [json.loads(l) for l in open("%s/runs/cli/logs/state_hashes.jsonl" % tmp)]
    assert [r["step"] for r in rows] == [0, 1, 2, 3, 4]


def test_safetensors_interchange_refuses_foreign_files_and_path_like_sidecar_names(tmp_path):
    """the header of an interchange file is untrusted input: a wrong format tag or a sidecar name that is not on the
    allow-list (anything path-like in particular) is refused before a single file is written"""
    import torch
    from safetensors.torch import save_file

    from open_transformers_b200.cli.dcp_safetensors import FORMAT, pack, unpack
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    res = train(tiny_cfg(tmp, ["train.ckpt_every_steps=2"]), device="cpu", data_root=tmp, max_steps=2)
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    info = pack(ck, str(tmp_path / "ok.safetensors"))
    assert "meta.json" in info["sidecar_files"] and "batch_hasher.rank_1.bin" in info["sidecar_files"]
    back = unpack(str(tmp_path / "ok.safetensors"), str(tmp_path / "back" / "checkpoints" / "step_000000002"))
    assert back["tensors"] == info["tensors"] and (tmp_path / "back" / "checkpoints" / "step_000000002" / "_COMPLETE").exists()
    t = {"model.w": torch.zeros(2)}
    skeleton = json.dumps({"t": "dict", "items": [["model", {"t": "dict", "items": [["w", {"t": "tensor", "key": "model.w"}]]}]]})
    save_file(t, str(tmp_path / "foreign.safetensors"), metadata={"pretrain.format": "something/9", "pretrain.skeleton": skeleton})
    with pytest.raises(ValueError):
        unpack(str(tmp_path / "foreign.safetensors"), str(tmp_path / "o1"))

    def sidecar(name):
        files = {"t": "dict", "items": [[name, {"t": "v", "v": "hi"}]]}
        return json.dumps({"t": "dict", "items": [["files", files], ["rng", {"t": "dict", "items": []}], ["grads", {"t": "v", "v": None}]]})

    for bad in ("../escape.txt", "/tmp/abs.txt", "sub/meta.json", "meta.json.bak", "rng.rank_x.pt"):
        save_file(t, str(tmp_path / "evil.safetensors"), metadata={"pretrain.format": FORMAT, "pretrain.skeleton": skeleton,
                                                                    "pretrain.sidecar": sidecar(bad)})
        with pytest.raises(ValueError):
            unpack(str(tmp_path / "evil.safetensors"), str(tmp_path / "o2"))
        assert not (tmp_path / "o2").exists() and not (tmp_path / "escape.txt").exists()
    save_file(t, str(tmp_path / "fine.safetensors"), metadata={"pretrain.format": FORMAT, "pretrain.skeleton": skeleton, "pretrain.sidecar": sidecar("meta.json")})
    unpack(str(tmp_path / "fine.safetensors"), str(tmp_path / "o3"))
    assert (tmp_path / "o3" / "meta.json").read_text() == "hi"
    with pytest.raises(FileNotFoundError):
        pack(str(tmp_path / "nowhere"), str(tmp_path / "x.safetensors"))


def test_tokenizer_isolates_digits_keeps_specials_and_hashes_canonically(corpus, tmp_path):
    from open_transformers_b200.data.tokenizer import SPECIAL_TOKENS, Tokenizer, compute_hash, train_tokenizer

    root, paths = corpus
    texts = [json.loads(l)["text"] for p in paths for l in open(p)]
    out = train_tokenizer(iter(texts), tmp_path / "t.json", vocab_size=330, min_frequency=1)
    tok = Tokenizer(out)
    assert [tok._tok.token_to_id(s) for s in SPECIAL_TOKENS] == list(range(6)) and tok.eos_id == 0
    assert len(tok.encode("6789")) == 4 and len(tok.encode("12")) == 2          # one token per digit, however frequent the number
    assert tok.decode(tok.encode("alpha 6789 beta")) == "alpha 6789 beta"
    assert tok.decode(tok.encode("héllo ☃")) == "héllo ☃"                        # bytes outside the training text still round-trip
    assert len(tok.encode_batch(["alpha", "beta gamma"])) == 2 and 256 < tok.vocab_size <= 330
    pretty = tmp_path / "pretty.json"                                            # the same tokenizer, re-serialised with other whitespace / key order
    pretty.write_text(json.dumps(json.loads(out.read_text()), indent=4, sort_keys=True, ensure_ascii=False))
    assert compute_hash(pretty) == compute_hash(out) == tok.hash


def test_doc_map_and_fetch_commands_and_a_replay_on_fetched_data(tmp_path, capsys):
    """the step -> document map from a config and from a checkpoint's position; the fetcher brings what the interval reads
    (verified) and stubs for the rest; the replay runs on the fetched copy, also when asked to fetch by itself"""
    import pyarrow.parquet as pq

    from open_transformers_b200.cli.audit_replay import main as audit_main
    from open_transformers_b200.cli.dump_doc_map import main as map_main
    from open_transformers_b200.cli.fetch_audit_data import main as fetch_main
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path / "origin")
    res = train(tiny_cfg(tmp, ["train.ckpt_every_steps=2"]), device="cpu", data_root=tmp)
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    over = ["train.seq_len=64", "data.seq_len=64", "model.max_seq_len_pretrain=64", "train.micro_batch_size=2",
            "train.global_batch_tokens.warmup=256", "train.global_batch_tokens.main=256", "train.global_batch_tokens.late=256"]
    # from step 0 to the checkpoint's step: chunk files, a manifest, and the position check against global_stream.json
    rc, out = _run(map_main, ["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "m0"), "--chunk-steps", "1"], capsys)
    man = json.loads((tmp_path / "m0" / "step_docs_manifest.json").read_text())
    rows0 = [r for f in man["files"] for r in pq.read_table(f).to_pylist()]
    assert rc == 0 and man["rows"] == len(rows0) > 0 and {r["step"] for r in rows0} == {0, 1} and man["validation"]["match"] is True
    assert [Path(f).name for f in man["files"]] == ["step_docs-000000-000000.parquet", "step_docs-000001-000001.parquet"]
    # a wrong topology override changes only the rank column; a walk that stops early is not compared
    rc, out = _run(map_main, ["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "m1"), "--until-step", "1", "--dp-world-size", "1"], capsys)
    man1 = json.loads((tmp_path / "m1" / "step_docs_manifest.json").read_text())
    assert rc == 0 and "validation" not in man1 and {r["dp_rank"] for f in man1["files"] for r in pq.read_table(f).to_pylist()} == {0}
    # from the checkpoint's own position: needs --until-step past it (this checkpoint carries no tokens over, or the tool
    # says why it cannot attribute them)
    with pytest.raises(SystemExit):
        map_main(["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "mx"), "--from-checkpoint-state"])
    with pytest.raises(SystemExit):
        map_main(["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "mx"), "--from-checkpoint-state", "--until-step", "2"])
    carry = json.loads((Path(ck) / "global_stream.json").read_text())["carry_over"]
    if carry:
        with pytest.raises(SystemExit):
            map_main(["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "m2"), "--from-checkpoint-state", "--until-step", "3"])
    else:
        rc, out = _run(map_main, ["--checkpoint", ck, "--data-root", tmp, "--out-dir", str(tmp_path / "m2"), "--from-checkpoint-state", "--until-step", "3"], capsys)
        rows2 = [r for f in json.loads((tmp_path / "m2" / "step_docs_manifest.json").read_text())["files"] for r in pq.read_table(f).to_pylist()]
        assert rc == 0 and {r["step"] for r in rows2} == {2}
    # a stream position that differs from the checkpoint's record exits 2
    doctored = tmp_path / "doctored"
    shutil.copytree(ck, doctored)
    gs = json.loads((doctored / "global_stream.json").read_text())
    gs["windows_emitted"] += 1
    (doctored / "global_stream.json").write_text(json.dumps(gs))
    rc, out = _run(map_main, ["--checkpoint", str(doctored), "--data-root", tmp, "--out-dir", str(tmp_path / "m3")], capsys)
    assert rc == 2 and json.loads((tmp_path / "m3" / "step_docs_manifest.json").read_text())["validation"]["match"] is False
    dest = tmp_path / "fetched"
    rc, out = _run(fetch_main, ["--checkpoint", ck, "--gcs-root", tmp, "--dest", str(dest), "--until-step", "3"], capsys)
    report = json.loads(out[:out.index("\nAudit this interval")])
    assert rc == 0 and report["data_root"] == str(dest) and report["verified"] and report["from_step"] == 2 and list(dest.rglob("manifest.yaml"))
    assert "--data-root %s" % dest in out
    rc, out = _run(fetch_main, ["--checkpoint", ck, "--mirror", tmp, "--dest", str(tmp_path / "unverified"), "--until-step", "3", "--no-verify",
                                "--config-name", "tiny_cpu"], capsys)
    assert rc == 0 and json.loads(out[:out.index("\nAudit this interval")])["verified"] is False
    assert audit_main(["--checkpoint", ck, "--data-root", str(dest), "--until-step", "3"]) == 0
    assert "MATCH=True" in capsys.readouterr().out
    # the replay fetching for itself: --gcs-root names the mirror, --fetch-dest where to put the interval's data
    assert audit_main(["--checkpoint", ck, "--gcs-root", tmp, "--fetch-dest", str(tmp_path / "auto"), "--until-step", "3"]) == 0
    assert "MATCH=True" in capsys.readouterr().out and list((tmp_path / "auto").rglob("*.bin"))


def test_overrides_and_options_may_come_in_any_order():
    import argparse

    from open_transformers_b200.cli._args import parse_with_overrides

    ap = argparse.ArgumentParser()
    ap.add_argument("--config-name", required=True)
    ap.add_argument("--flag", action="store_true")
    ap.add_argument("overrides", nargs="*")
    a = parse_with_overrides(ap, ["a.b=1", "--config-name", "x", "++c.d=[1,2]", "--flag", "~e.f", "+g=h=i"])
    assert a.config_name == "x" and a.flag and a.overrides == ["a.b=1", "++c.d=[1,2]", "~e.f", "+g=h=i"]
    for bad in (["--config-name", "x", "--nope"], ["a.b=1", "--config-name", "x", "loose_word"], ["a.b=1", "--config-name", "x", "=3"]):
        with pytest.raises(SystemExit):
            parse_with_overrides(ap, bad)


@pytest.mark.distributed
def test_launcher_script_runs_two_cpu_ranks_with_overrides_after_options(tmp_path):
    """scripts/launch_single_node.sh as documented: config, process count, then options and overrides in any order; two
    CPU ranks (gloo) write the hashes of the single-process run of the same recipe"""
    import os
    import subprocess
    from pathlib import Path

    from open_transformers_b200.train.loop import train

    root = Path(__file__).resolve().parent.parent
    tmp = str(tmp_path)
    over = ["model.n_layers=1", "train.total_tokens=768"]
    env = dict(os.environ, RUN_ID="launched", PYTHONPATH=str(root), OMP_NUM_THREADS="2", WANDB_MODE="disabled", MASTER_PORT="0")
    r = subprocess.run(["bash", str(root / "scripts" / "launch_single_node.sh"), "tiny_cpu", "2", "--synthetic-data", "--data-root", tmp, "--device", "cpu",
                        "run.output_dir=%s/runs" % tmp, *over], env=env, capture_output=True, text=True, timeout=600, cwd=str(root))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    got = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])["hashes"]
    from open_transformers_b200.config import load_config

    one = train(load_config("tiny_cpu", ["run.output_dir=%s/one" % tmp, "run.run_id=one", *over]), device="cpu", data_root=tmp)
    assert [tuple(h) for h in got] == [tuple(h) for h in one["hashes"]] and len(got) >= 1


def test_prepare_data_takes_the_reference_flag_forms(corpus, tmp_path, capsys):
    """--input-dir / --glob / --format inputs, fan-out sharding by byte range (--worker-id / --num-workers) joined by
    merge-manifests --output-dir, --shard-tag, inspect --shard --n, token-stats --tokenizer --sample, the configuration-free
    synthetic sources and replay-step --rank / --world-size / --seed / --override"""
    from open_transformers_b200.cli.prepare_data import main as prep
    from open_transformers_b200.data.indexed_dataset import IndexedDatasetReader
    from open_transformers_b200.data.manifest import SourceManifest

    root, paths = corpus
    tok_path = str(tmp_path / "tok.json")
    rc, out = _run(prep, ["train-tokenizer", "--input-dir", str(root), "--glob", "part*.jsonl", "--format", "jsonl", "--text-field", "text",
                          "--output", tok_path, "--vocab-size", "320", "--min-frequency", "1"], capsys)
    assert rc == 0 and Path(tok_path).exists()
    with pytest.raises(SystemExit):
        prep(["train-tokenizer", "--input-dir", str(root), "--glob", "*.nothing", "--output", tok_path])

    # one worker, then three workers over byte ranges of the same files: the same documents, in worker order
    one = tmp_path / "one"
    rc, out = _run(prep, ["shard", "--input-dir", str(root), "--glob", "part*.jsonl", "--format", "jsonl", "--tokenizer", tok_path, "--output-dir", str(one),
                          "--source-name", "src"], capsys)
    whole = SourceManifest.load(one / "manifest.yaml")
    assert rc == 0 and whole.total_documents == 120 and sorted(whole.raw_jsonl_blake2b) == ["part0.jsonl", "part1.jsonl"]
    fan = tmp_path / "fan"
    for k in range(3):
        rc, out = _run(prep, ["shard", "--input-dir", str(root), "--glob", "part*.jsonl", "--format", "jsonl", "--tokenizer", tok_path, "--output-dir", str(fan),
                              "--source-name", "src", "--worker-id", str(k), "--num-workers", "3"], capsys)
        assert rc == 0 and json.loads(out)["manifest"] == "manifest.w%02d.yaml" % k and list(fan.glob("src_w%02d_00000.bin" % k))
    with pytest.raises(SystemExit):
        prep(["merge-manifests", "--output-dir", str(fan), "--expected-workers", "4"])
    rc, out = _run(prep, ["merge-manifests", "--output-dir", str(fan), "--expected-workers", "3", "--remove-worker-manifests"], capsys)
    merged = SourceManifest.load(fan / "manifest.yaml")
    assert rc == 0 and merged.total_documents == 120 and merged.total_tokens == whole.total_tokens and not list(fan.glob("manifest.w*.yaml"))
    assert [s.prefix for s in merged.shards] == ["src_w00_00000", "src_w01_00000", "src_w02_00000"] and merged.raw_jsonl_blake2b == whole.raw_jsonl_blake2b

    def lengths(directory, man):
        return sorted(IndexedDatasetReader(directory / s.prefix).document_length(i) for s in man.shards for i in range(s.num_documents))

    assert lengths(fan, merged) == lengths(one, whole)
    with pytest.raises(SystemExit):
        prep(["shard", "--input-dir", str(root), "--glob", "part*.jsonl", "--tokenizer", tok_path, "--output-dir", str(fan), "--source-name", "src",
              "--num-workers", "2", "--shard-tag", "x"])
    rc, out = _run(prep, ["shard", str(paths[0]), "--tokenizer", tok_path, "--out-dir", str(tmp_path / "tagged"), "--name", "src", "--shard-tag", "w07"], capsys)
    assert rc == 0 and (tmp_path / "tagged" / "manifest.w07.yaml").exists() and (tmp_path / "tagged" / "src_w07_00000.bin").exists()

    rc, out = _run(prep, ["inspect", "--shard", str(one / whole.shards[0].prefix), "--tokenizer", tok_path, "--n", "2"], capsys)
    assert rc == 0 and len(json.loads(out)["samples"]) == 2
    sample = tmp_path / "sample.txt"
    sample.write_text("alpha beta gamma 12 345 " * 20, encoding="utf-8")
    rc, out = _run(prep, ["token-stats", "--tokenizer", tok_path, "--sample", str(sample)], capsys)
    assert rc == 0 and 1.0 < json.loads(out)["bytes_per_token"] < 10.0

    syn = tmp_path / "syn"
    rc, out = _run(prep, ["synthetic", "--output-dir", str(syn), "--docs-a", "40", "--docs-b", "20", "--min-doc-len", "8", "--max-doc-len", "32",
                          "--vocab-size", "500", "--seed", "3"], capsys)
    a, b = SourceManifest.load(syn / "synth_a" / "manifest.yaml"), SourceManifest.load(syn / "synth_b" / "manifest.yaml")
    assert rc == 0 and a.total_documents == 40 and b.total_documents == 20 and a.tokenizer_hash == "synthetic-no-tokenizer"
    r = IndexedDatasetReader(syn / "synth_a" / "synth_a_00000")
    docs = [r.document(i) for i in range(40)]
    assert all(8 <= len(d) <= 32 and 1 <= int(d.min()) and int(d.max()) < 500 for d in docs) and a.total_tokens == sum(len(d) for d in docs)

    data = str(tmp_path / "cfgdata")
    over = ["train.seq_len=64", "data.seq_len=64", "model.max_seq_len_pretrain=64", "train.micro_batch_size=2",
            "train.global_batch_tokens.warmup=256", "train.global_batch_tokens.main=256", "train.global_batch_tokens.late=256"]
    assert _run(prep, ["synthetic", "--config-name", "tiny_cpu", "--data-root", data, "--tokens", "4000", *over], capsys)[0] == 0
    rc, out = _run(prep, ["replay-step", "--config-name", "tiny_cpu", "--data-root", data, "--step", "1", "--override", *over], capsys)
    everyone = [json.loads(l) for l in out.splitlines()]
    rc, out = _run(prep, ["replay-step", "--config-name", "tiny_cpu", "--data-root", data, "--step", "1", "--rank", "1", "--world-size", "2", "--override", *over], capsys)
    rank1 = [json.loads(l) for l in out.splitlines()]
    assert rc == 0 and rank1 and {r["dp_rank"] for r in rank1} == {1} and rank1 == [r for r in everyone if r["dp_rank"] == 1]
    rc, out = _run(prep, ["replay-step", "--config-name", "tiny_cpu", "--data-root", data, "--step", "1", "--seed", "5", "--override", *over], capsys)
    assert rc == 0 and [json.loads(l)["tokens"] for l in out.splitlines()] != [r["tokens"] for r in everyone]
