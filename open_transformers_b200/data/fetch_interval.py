"""Fetch only the data an audit interval touches.

Given a checkpoint (its resolved config, stream position and step), the canonical stream is walked by
document LENGTHS - which needs the small ``.idx`` files and manifests only - to list the shards whose token
payload the interval reads. Those ``.bin`` files are downloaded and checked against the manifest's blake2b;
every other shard gets a sparse zero-length-on-disk stub of the right size so that readers can still mmap it.
The object store is reached through a *mirror* object (``exists/read_bytes/download``); ``GcsMirror`` wraps
google-cloud-storage when it is installed (anonymous client as fallback), ``DirMirror`` serves a local directory
(tests, air-gapped boxes) (reference src/pretrain/data/fetch_interval.py:60-534)."""
from __future__ import annotations

import json
import shutil
from pathlib import Path

from .manifest import SourceManifest, blake2b_file


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


def fetch_audit_interval(checkpoint: str | Path, mirror, dest: str | Path, until_step: int | None = None, cfg=None, *,
                         config_name: str | None = None, verify: bool = True) -> str:
    """Materialise under ``dest`` everything a replay of [checkpoint.step, until_step) needs; returns ``dest``.
    ``config_name``: a train config to use instead of the one recorded in the checkpoint; ``verify=False`` skips the
    blake2b comparison of downloaded files with their manifest (reference src/pretrain/cli/fetch_audit_data.py:49-60)."""
    from ..config import load_config, parse_config_resolved

    if cfg is None and config_name:
        cfg = load_config(config_name)

    if isinstance(mirror, str):
        mirror = GcsMirror(mirror) if mirror.startswith("gs://") else DirMirror(mirror)
    desc = read_checkpoint_descriptor(checkpoint)
    meta = desc["meta"]
    cfg = cfg or parse_config_resolved(meta["config_resolved"])
    dest = Path(dest)
    n_steps = (until_step - meta["step"]) if until_step else max(cfg.train.ckpt_every_steps, 1)
    # 1. manifests and indexes of every source (small)
    for src in cfg.data.sources:
        rel = Path(src.path)
        if not mirror.exists(str(rel / "manifest.yaml")):
            raise FileNotFoundError("mirror lacks %s" % (rel / "manifest.yaml"))
        mirror.download(str(rel / "manifest.yaml"), dest / rel / "manifest.yaml")
        man = SourceManifest.load(dest / rel / "manifest.yaml")
        for s in man.shards:
            mirror.download(str(rel / (s.prefix + ".idx")), dest / rel / (s.prefix + ".idx"))
            if verify and s.idx_blake2b and blake2b_file(dest / rel / (s.prefix + ".idx")) != s.idx_blake2b:
                raise FetchIntegrityError("%s.idx does not match its manifest digest" % s.prefix)
    # 2. which payloads are needed
    touched = enumerate_touched_shards(cfg, dest, desc["stream"], meta["consumed_tokens"], meta["step"], n_steps, meta["dp_world_size"])
    # 3. payloads: fetched + verified, or sparse stubs
    for src in cfg.data.sources:
        rel = Path(src.path)
        man = SourceManifest.load(dest / rel / "manifest.yaml")
        import numpy as np

        item = np.dtype(man.dtype).itemsize
        for sid, s in enumerate(man.shards):
            target = dest / rel / (s.prefix + ".bin")
            if sid in touched.get(man.name, set()):
                mirror.download(str(rel / (s.prefix + ".bin")), target)
                if verify and s.bin_blake2b and blake2b_file(target) != s.bin_blake2b:
                    target.unlink()
                    raise FetchIntegrityError("%s.bin does not match its manifest digest" % s.prefix)
            elif not target.exists():
                with open(target, "wb") as f:
                    f.truncate(s.token_count * item)   # sparse stub: right size, no blocks
    return str(dest)
