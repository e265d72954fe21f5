"""The canonical token stream: documents followed by the separator, cut into consecutive windows; a pure function of
(seed, sources, weights); mixing proportions; state round trip at an arbitrary point with carried-over tokens; epochs.
(reference test strategy: tests/test_global_stream.py, tests/test_mix_sampler.py, tests/test_checkpoint_global_stream.py)"""
import json

import numpy as np

from open_transformers_b200.data.global_stream import GlobalStream, GlobalStreamState
from open_transformers_b200.data.indexed_dataset import IndexedDatasetWriter
from open_transformers_b200.data.manifest import ShardInfo, SourceManifest, blake2b_file
from open_transformers_b200.data.mix_sampler import clear_caches


def _source(root, name, doc_token, n_docs, shards=2, seed=0):
    """A source whose every token equals ``doc_token`` + (document number % 7) * 1000, lengths 1..40."""
    rng = np.random.default_rng(seed)
    d = root / name
    d.mkdir(parents=True)
    infos, k = [], 0
    for s in range(shards):
        prefix = "shard_%05d" % s
        count = tokens = 0
        with IndexedDatasetWriter(d / prefix, np.uint32) as w:
            for _ in range(n_docs // shards):
                n = int(rng.integers(1, 41))
                w.add_document(np.full(n, doc_token + (k % 7) * 1000, dtype=np.uint32))
                k += 1; count += 1; tokens += n
        infos.append(ShardInfo(prefix, count, tokens, blake2b_file(d / (prefix + ".bin")), blake2b_file(d / (prefix + ".idx"))))
    man = SourceManifest(name=name, tokenizer_hash="none", dtype="uint32", shards=infos)
    man.save(d / "manifest.yaml")
    return man, str(d)


def _take(stream, n):
    it = iter(stream)
    return [next(it) for _ in range(n)]


def test_windows_are_documents_joined_by_the_separator(tmp_path):
    clear_caches()
    man, d = _source(tmp_path, "a", 5, 40)
    EOS, T = 3, 16
    windows = _take(GlobalStream([man], [d], [1.0], T, seed=9, eos_id=EOS), 20)
    assert all(w.shape == (T + 1,) and w.dtype == np.int64 for w in windows)
    flat = np.concatenate(windows)
    runs = np.split(flat, np.where(flat == EOS)[0] + 1)[:-1]      # complete documents, each ending with the separator
    assert len(runs) > 10
    for r in runs:
        body = r[:-1]
        assert 1 <= len(body) <= 40 and len(set(body.tolist())) == 1 and (body[0] - 5) % 1000 == 0
    again = _take(GlobalStream([man], [d], [1.0], T, seed=9, eos_id=EOS), 20)
    assert all(np.array_equal(a, b) for a, b in zip(windows, again))
    other = _take(GlobalStream([man], [d], [1.0], T, seed=10, eos_id=EOS), 20)
    assert not all(np.array_equal(a, b) for a, b in zip(windows, other))


def test_mixture_follows_the_document_weights(tmp_path):
    clear_caches()
    a, da = _source(tmp_path, "a", 5, 400, seed=1)
    b, db = _source(tmp_path, "b", 6, 400, seed=2)
    EOS = 3
    flat = np.concatenate(_take(GlobalStream([a, b], [da, db], [3.0, 1.0], 64, seed=4, eos_id=EOS), 120))
    docs = np.split(flat, np.where(flat == EOS)[0] + 1)[:-1]
    from_a = sum(1 for r in docs if len(r) > 1 and (r[0] - 5) % 1000 == 0)
    from_b = sum(1 for r in docs if len(r) > 1 and (r[0] - 6) % 1000 == 0)
    assert from_a + from_b == len(docs) and 0.68 < from_a / len(docs) < 0.82      # weights are per DOCUMENT draws: 3 : 1


def test_state_round_trip_mid_document_and_across_an_epoch(tmp_path):
    clear_caches()
    man, d = _source(tmp_path, "a", 5, 20)                  # 20 documents: the stream wraps into new epochs quickly
    T, EOS = 24, 3
    ref = _take(GlobalStream([man], [d], [1.0], T, seed=2, eos_id=EOS), 60)
    for cut in (1, 7, 33):
        s = GlobalStream([man], [d], [1.0], T, seed=2, eos_id=EOS)
        it = iter(s)
        for _ in range(cut):
            next(it)
        state = GlobalStreamState.from_json(json.loads(json.dumps(s.state().to_json())))     # through the checkpoint's JSON
        assert state.windows_emitted == cut
        resumed = _take(GlobalStream([man], [d], [1.0], T, seed=2, eos_id=EOS, state=state), 60 - cut)
        assert all(np.array_equal(x, y) for x, y in zip(resumed, ref[cut:])), cut
    s = GlobalStream([man], [d], [1.0], T, seed=2, eos_id=EOS)
    _take(s, 60)
    st = s.state()
    assert st.epoch_per_source["a"] >= 1 and 0 <= st.consumed_documents_per_source["a"] < 20
    assert len(st.carry_over) < 42                              # less than one document plus its separator is ever buffered


def test_every_document_appears_once_per_epoch(tmp_path):
    clear_caches()
    rng = np.random.default_rng(0)
    d = tmp_path / "u"
    d.mkdir()
    with IndexedDatasetWriter(d / "shard_00000", np.uint32) as w:
        for i in range(30):
            w.add_document(np.full(int(rng.integers(2, 9)), 100 + i, dtype=np.uint32))
    man = SourceManifest(name="u", tokenizer_hash="none", dtype="uint32", shards=[ShardInfo("shard_00000", 30, 0, blake2b_file(d / "shard_00000.bin"),
                                                                            blake2b_file(d / "shard_00000.idx"))])
    flat = np.concatenate(_take(GlobalStream([man], [str(d)], [1.0], 32, seed=1, eos_id=0), 40))
    ids = [int(r[0]) for r in np.split(flat, np.where(flat == 0)[0] + 1)[:-1]]
    first, second = ids[:30], ids[30:60]
    assert sorted(first) == list(range(100, 130)) and sorted(second) == list(range(100, 130)) and first != second


def test_token_share_weights_become_document_probabilities(tmp_path):
    """``weights_are_token_shares``: a source with documents ten times longer gets a tenth of the document draws per
    unit of weight, so that the TOKEN shares of the stream follow the weights"""
    import types

    from open_transformers_b200.data.loader import resolve_sources

    clear_caches()
    rng = np.random.default_rng(0)
    mans = []
    for name, tok, length in (("short", 5, 8), ("long", 6, 80)):
        d = tmp_path / name
        d.mkdir()
        with IndexedDatasetWriter(d / "shard_00000", np.uint32) as w:
            for _ in range(300):
                w.add_document(np.full(length, tok, dtype=np.uint32))
        man = SourceManifest(name=name, tokenizer_hash="none", dtype="uint32",
                             shards=[ShardInfo("shard_00000", 300, 300 * length, blake2b_file(d / "shard_00000.bin"), blake2b_file(d / "shard_00000.idx"))])
        man.save(d / "manifest.yaml")
        mans.append(man)

    def data_cfg(token_shares):
        srcs = [types.SimpleNamespace(name="short", path="short", weight=1.0), types.SimpleNamespace(name="long", path="long", weight=1.0)]
        return types.SimpleNamespace(sources=srcs, weights_are_token_shares=token_shares, normalised_weights=lambda: [0.5, 0.5])

    _, dirs, w_doc = resolve_sources(data_cfg(False), str(tmp_path))
    _, _, w_tok = resolve_sources(data_cfg(True), str(tmp_path))
    assert w_doc == [0.5, 0.5] and abs(w_tok[0] - 10 / 11) < 1e-12 and abs(sum(w_tok) - 1) < 1e-12
    flat = np.concatenate(_take(GlobalStream(mans, dirs, w_tok, 64, seed=3, eos_id=0), 400))
    share_short = float((flat == 5).sum()) / float(((flat == 5) | (flat == 6)).sum())
    assert 0.42 < share_short < 0.58                      # equal TOKEN shares, as the weights say


def test_legacy_per_rank_sampler_is_strided_resumable_and_topology_dependent(tmp_path):
    """the legacy sampler (DDP runs): ranks walk disjoint strides of each source's permutation, the state round-trips, and
    - unlike the canonical stream - the windows depend on the world size"""
    from open_transformers_b200.data.mix_sampler import MixSampler, MixSamplerState

    clear_caches()
    man, d = _source(tmp_path, "a", 5, 40)
    two = [_take(MixSampler([man], [d], [1.0], 16, seed=4, rank=r, world_size=2, eos_id=3), 6) for r in range(2)]
    again = _take(MixSampler([man], [d], [1.0], 16, seed=4, rank=1, world_size=2, eos_id=3), 6)
    assert all(np.array_equal(a, b) for a, b in zip(two[1], again))
    assert not all(np.array_equal(a, b) for a, b in zip(two[0], two[1]))
    one = _take(MixSampler([man], [d], [1.0], 16, seed=4, rank=0, world_size=1, eos_id=3), 6)
    assert not all(np.array_equal(a, b) for a, b in zip(one, two[0]))
    s = MixSampler([man], [d], [1.0], 16, seed=4, rank=0, world_size=2, eos_id=3)
    it = iter(s)
    for _ in range(3):
        next(it)
    st = MixSamplerState(**json.loads(json.dumps(s.state().__dict__)))
    rest = _take(MixSampler([man], [d], [1.0], 16, seed=4, rank=0, world_size=2, eos_id=3, state=st), 3)
    assert all(np.array_equal(a, b) for a, b in zip(rest, two[0][3:]))


def test_text_iterators_read_jsonl_parquet_and_byte_segments(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq

    from open_transformers_b200.data.prepare import iter_jsonl, iter_jsonl_segment, iter_parquet, iter_texts

    texts = ["doc %d %s" % (i, "x" * (i % 7)) for i in range(50)]
    j = tmp_path / "a.jsonl"
    j.write_text("\n".join(json.dumps({"text": t, "other": i}) for i, t in enumerate(texts)) + "\n")
    p = tmp_path / "b.parquet"
    pq.write_table(pa.table({"text": texts[::-1], "n": list(range(50))}), p)
    assert list(iter_jsonl(j)) == texts and list(iter_parquet(p, batch_size=7)) == texts[::-1]
    assert list(iter_texts([j, p])) == texts + texts[::-1]
    size = j.stat().st_size
    for cuts in ([0, size], [0, 1, size], [0, size // 3, size // 2, size - 1, size], [0, 17, 18, 19, size]):
        got = [t for a, b in zip(cuts[:-1], cuts[1:]) for t in iter_jsonl_segment(j, a, b)]
        assert got == texts, cuts                    # every line belongs to exactly one segment, wherever the cuts fall
