import numpy as np
import pytest

from open_transformers_b200.data.indexed_dataset import IndexedDatasetReader, IndexedDatasetWriter, MAGIC
from open_transformers_b200.data.loader import build_global_loader, build_global_stream
from open_transformers_b200.data.manifest import SourceManifest, blake2b_file
from open_transformers_b200.data.mix_sampler import SourceWalker, clear_caches
from open_transformers_b200.train.batch_schedule import (accum_for_rank, iter_step_plans, microbatches_per_step, owner_rank,
                                                         windows_consumed_before)
from helpers import tiny_cfg


def test_indexed_dataset_round_trip(tmp_path):
    docs = [np.arange(5), np.array([], dtype=np.int64), np.array([7, 8, 9])]
    with IndexedDatasetWriter(tmp_path / "s", np.uint16) as w:
        for d in docs:
            w.add_document(d)
    raw = (tmp_path / "s.idx").read_bytes()
    assert raw[:8] == MAGIC and len(raw) == 33 + 16 * 4
    r = IndexedDatasetReader(tmp_path / "s")
    assert r.num_documents == 3 and r.token_count == 8 and r.dtype == np.uint16
    for i, d in enumerate(docs):
        assert np.array_equal(r.document(i), d) and r.document_length(i) == len(d)
    ro = IndexedDatasetReader(tmp_path / "s", index_only=True)
    assert ro.document_length(2) == 3
    with pytest.raises(RuntimeError):
        ro.document(0)
    (tmp_path / "bad.idx").write_bytes(b"NOTMAGIC" + raw[8:])
    with pytest.raises(ValueError):
        IndexedDatasetReader(tmp_path / "bad", index_only=True)


def test_manifest_hashes_and_verify(tmp_path):
    cfg = tiny_cfg(str(tmp_path))
    src = tmp_path / cfg.data.sources[0].path
    man = SourceManifest.load(src / "manifest.yaml")
    assert man.total_tokens > 0 and man.verify(src) == []
    p = src / (man.shards[0].prefix + ".bin")
    data = bytearray(p.read_bytes()); data[0] ^= 1; p.write_bytes(bytes(data))
    assert man.verify(src) == [str(p)]
    assert len(blake2b_file(p)) == 64


def test_walker_permutation_is_a_permutation_and_strided(tmp_path):
    cfg = tiny_cfg(str(tmp_path))
    src = tmp_path / cfg.data.sources[0].path
    man = SourceManifest.load(src / "manifest.yaml")
    clear_caches()
    full = SourceWalker(man, str(src), seed=3)
    order = [full.next_document_ref() for _ in range(full.total_documents)]
    assert len(set(order)) == full.total_documents
    a, b = SourceWalker(man, str(src), 3, 0, 2), SourceWalker(man, str(src), 3, 1, 2)
    assert [a.next_document_ref() for _ in range(5)] == order[0:10:2] and [b.next_document_ref() for _ in range(5)] == order[1:10:2]
    full.next_document_ref()
    assert full.epoch == 1  # wrapped into the next epoch with a new permutation


def test_sharded_view_equals_global_stream_for_any_split(tmp_path):
    cfg = tiny_cfg(str(tmp_path))
    it = iter(build_global_stream(cfg, data_root=str(tmp_path)))
    windows = [next(it) for _ in range(12)]
    for world_ranks in ([[0, 1]], [[0], [1]]):
        seen = {}
        for ranks in world_ranks:
            view = iter(build_global_loader(cfg, ranks, 2, data_root=str(tmp_path)))
            for step in range(3):
                plan, batches = next(view)
                for r, k, w in batches:
                    m = k * 2 + r
                    for slot in range(cfg.train.micro_batch_size):
                        seen[plan.base_window + m * cfg.train.micro_batch_size + slot] = w[slot]
        assert sorted(seen) == list(range(12))
        for i in range(12):
            assert np.array_equal(seen[i], windows[i])


def test_stream_state_resume(tmp_path):
    cfg = tiny_cfg(str(tmp_path))
    view = build_global_loader(cfg, [0, 1], 2, data_root=str(tmp_path))
    it = iter(view)
    next(it)
    state, (step, consumed, _) = view.state(), view.position
    want = next(it)[1]
    resumed = build_global_loader(cfg, [0, 1], 2, state=state, consumed_tokens=consumed, start_step=step, data_root=str(tmp_path))
    got = next(iter(resumed))[1]
    assert all(np.array_equal(a[2], b[2]) for a, b in zip(want, got))
    assert state.windows_emitted == windows_consumed_before(consumed, cfg.train)


def test_batch_schedule_math():
    from open_transformers_b200.config import load_config

    tr = load_config("1b_repop_v2").train
    assert microbatches_per_step(0, tr) == 192 and microbatches_per_step(5_000_000_000, tr) == 288 and microbatches_per_step(370_000_000_000, tr) == 576
    assert [owner_rank(m, world_size=4) for m in range(6)] == [0, 1, 2, 3, 0, 1]
    assert sum(accum_for_rank(10, world_size=4, rank=r) for r in range(4)) == 10
    plans = iter_step_plans(0, 0, tr)
    p0, p1 = next(plans), next(plans)
    assert p1.base_window == p0.microbatches * tr.micro_batch_size and p1.consumed_tokens == p0.tokens_this_step


def test_corpus_fan_out_shards_every_document_once_in_file_order(tmp_path):
    """scripts/build_corpus.py: bucket shuffle is a permutation, and the parallel sharding fan-out writes every
    document exactly once, in file order across the worker directories, with a merged manifest that reads back."""
    import json
    import sys
    from pathlib import Path

    from open_transformers_b200.data.indexed_dataset import IndexedDatasetReader
    from open_transformers_b200.data.manifest import SourceManifest
    from open_transformers_b200.data.tokenizer import Tokenizer, train_tokenizer

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "scripts"))  # the workers import the module by name
    import build_corpus as bc
    docs = ["document number %d says hello %s" % (i, "x" * (i % 7)) for i in range(101)]
    src = tmp_path / "c.jsonl"
    src.write_text("\n".join(json.dumps({"text": d}) for d in docs) + "\n")
    shuffled = tmp_path / "s.jsonl"
    assert bc.shuffle_jsonl(str(src), str(shuffled), seed=3, n_buckets=8) == 101
    assert sorted(shuffled.read_text().splitlines()) == sorted(src.read_text().splitlines())
    assert shuffled.read_text() != src.read_text()
    tok_path = train_tokenizer(iter(docs), tmp_path / "tok.json", vocab_size=300, min_frequency=1)
    man = bc.shard_source(str(src), str(tok_path), str(tmp_path / "out"), "toy", workers=3, shard_bytes=1 << 20)
    assert man.total_documents == 101
    back = SourceManifest.load(tmp_path / "out" / "manifest.yaml")
    tok, seen = Tokenizer(tok_path), []
    for sh in back.shards:
        r = IndexedDatasetReader(str(tmp_path / "out" / sh.prefix))
        seen += [tok.decode(r.document(i).tolist()) for i in range(sh.num_documents)]
    assert seen == docs


def test_corpus_pulls_resume_where_they_stopped_and_the_build_stages_are_idempotent(tmp_path):
    """scripts/build_corpus.py with stand-ins for the network: a pull that dies between two resume notes is cut back to the
    last note and continues from the recorded row of the raw stream (a filter that drops three rows in four makes the two
    counts differ), quotas split a target over several configurations, file lists are visited round-robin without their
    evaluation splits, blob fetches keep their order, and `build` skips what is already there."""
    import json
    import sys
    from pathlib import Path

    from open_transformers_b200.data.manifest import SourceManifest
    from open_transformers_b200.data.tokenizer import train_tokenizer

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "scripts"))
    import build_corpus as bc

    calls = []

    def rows(skip):
        calls.append(skip)
        for i in range(skip, 100_000):
            yield {"text": "row %d" % i, "int_score": 3 if i % 4 == 0 else 1}

    keep = lambda r: r["text"] if r["int_score"] >= 3 else None  # noqa: E731
    out = tmp_path / "raw" / "fineweb.jsonl"

    class Died(Exception):
        pass

    def dying(skip):
        for r in rows(skip):
            if r["text"] == "row 1000":       # the 251st kept row: past the note written at 200 documents
                raise Died()
            yield r

    with pytest.raises(Died):
        bc.pull(out, 500, [(bc.Stream("fw", dying, keep), None)], chunk=100)
    assert len(out.read_text().splitlines()) == 250 and json.loads((tmp_path / "raw" / "fineweb.jsonl.scanned").read_text())["taken"] == {"fw": 200}
    with open(out, "a") as f:
        f.write('{"text": "torn li')                                         # and a torn last line on top
    have, scanned = bc.pull(out, 500, [(bc.Stream("fw", rows, keep), None)], chunk=100)
    texts = [json.loads(l)["text"] for l in out.read_text().splitlines()]
    assert have == 500 and texts == ["row %d" % (4 * i) for i in range(500)]  # nothing lost, nothing twice
    assert calls[-1] == 797 and scanned == {"fw": 1997}                       # resumed at the raw row after the 200th kept one
    assert bc.pull(out, 500, [(bc.Stream("fw", rows, keep), None)], chunk=100)[0] == 500 and len(out.read_text().splitlines()) == 500
    (tmp_path / "raw" / "fineweb.jsonl.scanned").write_text(json.dumps({"taken": {"fw": 900}, "scanned": {"fw": 1}}))
    with pytest.raises(RuntimeError):
        bc.pull(out, 1000, [(bc.Stream("fw", rows, keep), None)], chunk=100)

    shares = bc.split_by_weight(1001, {"a": 0.5, "b": 0.3, "c": 0.2})
    assert shares == {"a": 500, "b": 300, "c": 201}
    mixed = tmp_path / "raw" / "proof.jsonl"
    streams = [(bc.Stream(k, (lambda k: lambda skip: ({"text": "%s %d" % (k, i)} for i in range(skip, 10_000)))(k), bc.text_of), q) for k, q in shares.items()]
    assert bc.pull(mixed, 1001, streams, chunk=100)[0] == 1001
    kinds = [json.loads(l)["text"].split()[0] for l in mixed.read_text().splitlines()]
    assert kinds == ["a"] * 500 + ["b"] * 300 + ["c"] * 201

    order = [p for _, p in bc.round_robin_files({"math": ["m1", "m2", "m3"], "code": ["c1"], "web": ["w1", "w2"]})]
    assert order == ["c1", "m1", "w1", "m2", "w2", "m3"]
    assert bc.is_eval_split("/data/math/test/part-0.jsonl") and bc.is_eval_split("/x/heldout-1.jsonl") and not bc.is_eval_split("/data/math/train/part-0.jsonl")
    import time as _t

    fetched = list(bc.ordered_fetch(range(40), lambda i: (_t.sleep(0.001 * (i % 5)), None if i % 7 == 0 else i * i)[1], workers=8, window=16))
    assert [i for i, _ in fetched] == list(range(40)) and fetched[7] == (7, None) and fetched[6] == (6, 36)
    stack = bc.source_streams("stack", 10, fetch_blob=lambda r: "code of " + r["blob_id"], workers=4)
    assert len(stack) == 1 and stack[0][1] is None

    docs = ["document number %d says hello" % i for i in range(300)]
    tok = train_tokenizer(iter(docs), tmp_path / "tok.json", vocab_size=300, min_frequency=1)
    pulled = []

    def fake_pull(raw, n, source):
        pulled.append(source)
        Path(raw).parent.mkdir(parents=True, exist_ok=True)
        Path(raw).write_text("".join(json.dumps({"text": d}) + "\n" for d in docs[:n]))
        return n, {}

    done = bc.build({"dclm": 120, "proof": 0, "fineweb": 80}, tmp_path / "r", tmp_path / "s", tok, workers=2, only=["dclm", "fineweb"], pull_fn=fake_pull, log=lambda m: None)
    assert pulled == ["dclm", "fineweb"] and set(done) == {"dclm", "fineweb"}
    man = SourceManifest.load(done["dclm"])
    assert man.total_documents == 120 and man.name == "dclm_baseline" and (tmp_path / "r" / "dclm_baseline.jsonl.shuffled").is_file()
    assert done["dclm"] == str(tmp_path / "s" / "dclm_baseline_proxy" / "manifest.yaml")       # the directory the data recipes name
    assert sorted(json.loads(l)["text"] for l in (tmp_path / "r" / "dclm_baseline.jsonl").read_text().splitlines()) == sorted(docs[:120])
    again = bc.build({"dclm": 120, "fineweb": 80}, tmp_path / "r", tmp_path / "s", tok, workers=2, pull_fn=fake_pull, log=lambda m: None)
    assert again == done and pulled == ["dclm", "fineweb"]                   # manifests exist: nothing pulled or sharded again
    # the recipes' long names select sources too; a midtraining source is built only when named; a Stack fan-out worker writes
    # tagged files that merge-manifests joins
    assert bc.build({"dclm": 5, "dolma3_dolmino_mix": 5}, tmp_path / "r2", tmp_path / "s2", tok, workers=1, only=["dclm_baseline"], pull_fn=fake_pull,
                    log=lambda m: None).keys() == {"dclm"}
    assert "dolma3_dolmino_mix" not in bc.build({"dolma3_dolmino_mix": 5}, tmp_path / "r2", tmp_path / "s2", tok, workers=1, pull_fn=fake_pull, log=lambda m: None)
    with pytest.raises(ValueError):
        bc.build({"dclm": 5}, tmp_path / "r3", tmp_path / "s3", tok, workers=1, only=["dclm"], pull_fn=fake_pull, log=lambda m: None, num_workers=2)
    for k in range(2):
        part = bc.build({"stack": 40}, tmp_path / "r3", tmp_path / "s3", tok, suffix="", workers=1, only=["stack_v2_permissive"], pull_fn=fake_pull,
                        log=lambda m: None, worker_id=k, num_workers=2)
        assert part["stack"].endswith("stack_v2_permissive/manifest.w%02d.yaml" % k) and (tmp_path / "r3" / ("stack_v2_permissive_w%02d.jsonl" % k)).is_file()
    from open_transformers_b200.data.prepare import merge_worker_manifests

    merged = merge_worker_manifests(tmp_path / "s3" / "stack_v2_permissive", expected_workers=2)
    assert merged.total_documents == 80 and merged.name == "stack_v2_permissive" and all(s.prefix.startswith(("w00/", "w01/")) for s in merged.shards)
