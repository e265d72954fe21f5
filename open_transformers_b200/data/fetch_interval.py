"""Fetch only the data an audit interval touches.

Given a checkpoint (its resolved config, stream position and step), the canonical stream is walked by
document LENGTHS - which needs the small ``.idx`` files and manifests only - to list the shards whose token
payload the interval reads. Those ``.bin`` files are downloaded and checked against the manifest's blake2b;
every other shard gets a sparse zero-length-on-disk stub of the right size so that readers can still mmap it.
The object store is reached through a *mirror* object (``exists/read_bytes/download``); ``GcsMirror`` wraps
google-cloud-storage when it is installed (anonymous client as fallback), ``DirMirror`` serves a local directory
(tests, air-gapped boxes) (reference src/pretrain/data/fetch_interval.py:60-534)."""
from __future__ import annotations

import dataclasses
import json
import logging
import shutil
from pathlib import Path

import numpy as np

from .manifest import SourceManifest, blake2b_file

log = logging.getLogger("pretrain.fetch_interval")


class DirMirror:
    def __init__(self, root: str | Path):
        self.root = Path(root)

    def exists(self, rel: str) -> bool:
        return (self.root / rel).is_file()

    def read_bytes(self, rel: str) -> bytes:
        return (self.root / rel).read_bytes()

    def download(self, rel: str, dest: str | Path) -> None:
        Path(dest).parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(self.root / rel, dest)


class GcsMirror:
    def __init__(self, gcs_root: str):
        if not gcs_root.startswith("gs://"):
            raise ValueError("gcs root must look like gs://bucket/prefix")
        bucket, _, prefix = gcs_root[5:].partition("/")
        try:
            from google.cloud import storage  # type: ignore
        except Exception as e:
            raise RuntimeError("google-cloud-storage is not installed; pass a local mirror directory instead") from e
        try:
            client = storage.Client()
        except Exception:
            client = storage.Client.create_anonymous_client()
        self._bucket, self._prefix = client.bucket(bucket), prefix.rstrip("/")

    def _blob(self, rel):
        return self._bucket.blob("%s/%s" % (self._prefix, rel) if self._prefix else rel)

    def exists(self, rel):
        return self._blob(rel).exists()

    def read_bytes(self, rel):
        return self._blob(rel).download_as_bytes()

    def download(self, rel, dest):
        Path(dest).parent.mkdir(parents=True, exist_ok=True)
        self._blob(rel).download_to_filename(str(dest))


class FetchIntegrityError(RuntimeError):
    pass


def read_checkpoint_descriptor(ckpt_dir: str | Path) -> dict:
    d = Path(ckpt_dir)
    meta = json.loads((d / "meta.json").read_text())
    stream = json.loads((d / "global_stream.json").read_text()) if (d / "global_stream.json").exists() else None
    return {"meta": meta, "stream": stream}


def enumerate_touched_shards(cfg, data_root: str | Path, stream_state, consumed_tokens: int, start_step: int, n_steps: int, dp_world_size: int):
    """{source name: set(shard ids)} read by steps [start_step, start_step + n_steps)."""
    from .global_stream import GlobalStreamState, ShardedWindowView
    from .loader import resolve_sources
    from .mix_sampler import clear_caches

    clear_caches()
    manifests, dirs, weights = resolve_sources(cfg.data, str(data_root))
    state = GlobalStreamState.from_json(stream_state) if isinstance(stream_state, dict) else stream_state
    view = ShardedWindowView.__new__(ShardedWindowView)
    from .global_stream import _Core

    literal_ok = state is None or not state.carry_over
    view._core = _Core(manifests, dirs, weights, cfg.data.seq_len, cfg.run.seed, cfg.data.document_separator_id, state, index_only=True)
    view.train, view.world_size, view.ranks = cfg.train, dp_world_size, []
    view._consumed_tokens, view._step = consumed_tokens, start_step
    touched: dict[str, set] = {}
    for _step, _m, _slot, source, shard, *_ in view.walk_doc_refs(n_steps):
        touched.setdefault(source, set()).add(int(shard))
    clear_caches()
    return touched


@dataclasses.dataclass
class FetchResult:
    dest: str
    data_root: str                       # what the replay takes as --data-root
    start_step: int
    start_consumed_tokens: int
    until_step: int
    from_init: bool
    touched_shards: dict                 # {source name: sorted shard ids}
    bytes_fetched: int                   # payload bytes that landed on disk in this call (0 for shards already present and verified)
    stubs_created: int
    verified: bool


def _fetch_indices(mirror, rel: Path, dest: Path, verify: bool) -> SourceManifest:
    """A source's manifest and every shard's ``.idx`` (a fraction of a percent of the corpus): what the length walk needs.
    Index files already present are kept when they match the manifest's digest."""
    if not mirror.exists(str(rel / "manifest.yaml")):
        raise FileNotFoundError("mirror lacks %s" % (rel / "manifest.yaml"))
    mirror.download(str(rel / "manifest.yaml"), dest / rel / "manifest.yaml")
    man = SourceManifest.load(dest / rel / "manifest.yaml")
    for s in man.shards:
        idx = dest / rel / (s.prefix + ".idx")
        if not idx.exists() or (verify and s.idx_blake2b and blake2b_file(idx) != s.idx_blake2b):
            mirror.download(str(rel / (s.prefix + ".idx")), idx)
        if verify and s.idx_blake2b and blake2b_file(idx) != s.idx_blake2b:
            raise FetchIntegrityError("%s does not match its manifest digest: the mirror is corrupt or stale for this shard" % idx)
    return man


def _fetch_payloads(mirror, rel: Path, dest: Path, man: SourceManifest, shard_ids, verify: bool) -> int:
    """The whole ``.bin`` of every touched shard, checked against the manifest's blake2b - a stronger statement than a
    replay (the bytes ARE the cluster's). A file already there is kept if it verifies; a sparse stub left by an earlier,
    shorter fetch fails the digest and is replaced. Returns the bytes downloaded."""
    fetched = 0
    for sid in sorted(shard_ids):
        s = man.shards[sid]
        target = dest / rel / (s.prefix + ".bin")
        if target.exists():
            size_ok = target.stat().st_size == s.token_count * np.dtype(man.dtype).itemsize
            if size_ok and (not verify or not s.bin_blake2b or blake2b_file(target) == s.bin_blake2b) and not _is_sparse_stub(target):
                continue
            target.unlink()
        mirror.download(str(rel / (s.prefix + ".bin")), target)
        fetched += target.stat().st_size
        if verify and s.bin_blake2b and blake2b_file(target) != s.bin_blake2b:
            target.unlink()
            raise FetchIntegrityError("%s.bin does not match its manifest digest: the mirror is corrupt or stale for this shard" % s.prefix)
    return fetched


def _is_sparse_stub(path: Path) -> bool:
    """A placeholder written by ``_stub_untouched``: a file with bytes but no blocks. (Only consulted when verification is
    off or the manifest has no digest; with a digest the zeros fail the comparison anyway.)"""
    st = path.stat()
    return st.st_size > 0 and getattr(st, "st_blocks", 1) == 0


def _stub_untouched(dest: Path, rel: Path, man: SourceManifest, touched: set) -> int:
    """The loader opens a reader for EVERY shard of every source, and a payload reader wants its ``.bin`` to exist. Shards the
    interval never reads get a sparse file of the right size (no disk blocks); were the walk ever to read one, the zeros
    would surface as a hash mismatch, not as silent corruption."""
    item, made = np.dtype(man.dtype).itemsize, 0
    for sid, s in enumerate(man.shards):
        target = dest / rel / (s.prefix + ".bin")
        if sid in touched or target.exists():
            continue
        with open(target, "wb") as f:
            f.truncate(s.token_count * item)
        made += 1
    return made


def fetch_audit_interval(checkpoint: str | Path, mirror, dest: str | Path = "./data/audit_data", until_step: int | None = None, cfg=None, *,
                         config_name: str | None = None, from_init: bool = False, verify: bool = True) -> FetchResult:
    """Materialise under ``dest`` everything a replay of the interval that starts at ``checkpoint`` needs.

    The interval ends at ``until_step``, by default one checkpoint interval after the start (``ckpt_every_steps``, or the
    first step across the next multiple of ``ckpt_every_tokens``). ``from_init=True`` matches ``audit_replay --from-init``:
    the walk starts at the ORIGIN of the canonical stream (step 0, fresh state) and runs to ``until_step`` (default: the
    checkpoint's own step); the checkpoint then only supplies configuration, seed and topology. ``config_name``: a train
    configuration to use instead of the recorded one; ``verify=False`` skips the blake2b comparisons. A second call with
    a longer interval keeps verified files and replaces the stubs that became touched. Writes ``fetch_manifest.json``.
    (reference src/pretrain/data/fetch_interval.py:393-534)"""
    from ..config import load_config, parse_config_resolved
    from ..train.batch_schedule import default_interval_end

    if isinstance(mirror, str):
        mirror = GcsMirror(mirror) if mirror.startswith("gs://") else DirMirror(mirror)
    desc = read_checkpoint_descriptor(checkpoint)
    meta = desc["meta"]
    if cfg is None:
        cfg = load_run_config(meta, config_name)
    dest = Path(dest)
    if from_init:
        stream, start_step, start_consumed = None, 0, 0
        until_step = int(meta["step"]) if until_step is None else until_step
    else:
        stream, start_step, start_consumed = desc["stream"], int(meta["step"]), int(meta["consumed_tokens"])
        if until_step is None:
            until_step = default_interval_end(start_step, start_consumed, cfg.train)
    if until_step <= start_step:
        raise ValueError("until_step %d is not beyond the starting step %d" % (until_step, start_step))
    log.info("fetch interval: step %d (%d tokens) -> step %d, seed %s%s", start_step, start_consumed, until_step, meta.get("seed"),
             " (from the stream's origin)" if from_init else "")
    # 1. manifests and indexes of every source (small)
    manifests = {}
    for src in cfg.data.sources:
        manifests[src.path] = _fetch_indices(mirror, Path(src.path), dest, verify)
    # 2. which payloads the interval reads: the same window cursor the replay drives, over document lengths only
    touched = enumerate_touched_shards(cfg, dest, stream, start_consumed, start_step, until_step - start_step, int(meta.get("dp_world_size") or 1))
    log.info("interval touches %d shard(s) of %d source(s): %s", sum(len(v) for v in touched.values()), len(touched),
             {k: len(v) for k, v in touched.items()})
    # 3. payloads, then sparse stand-ins for everything else
    fetched = stubs = 0
    for src in cfg.data.sources:
        man = manifests[src.path]
        ids = touched.get(man.name, set())
        fetched += _fetch_payloads(mirror, Path(src.path), dest, man, ids, verify)
        stubs += _stub_untouched(dest, Path(src.path), man, ids)
    log.info("downloaded %.2f GB of shard payloads, %d sparse placeholder(s) for untouched shards", fetched / 1e9, stubs)
    result = FetchResult(dest=str(dest), data_root=str(dest), start_step=start_step, start_consumed_tokens=start_consumed, until_step=until_step,
                         from_init=from_init, touched_shards={k: sorted(v) for k, v in touched.items()}, bytes_fetched=fetched,
                         stubs_created=stubs, verified=verify)
    (dest / "fetch_manifest.json").write_text(json.dumps(dataclasses.asdict(result), indent=2) + "\n")
    return result


def load_run_config(meta: dict, config_name: str | None = None):
    """The run's configuration: a named one when given, else the one embedded in the checkpoint's metadata."""
    from ..config import load_config, parse_config_resolved

    if config_name:
        return load_config(config_name)
    if not meta.get("config_resolved"):
        raise ValueError("the checkpoint embeds no configuration; pass config_name")
    return parse_config_resolved(meta["config_resolved"])
