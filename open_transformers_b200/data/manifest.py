"""Per-source shard manifest: ``manifest.yaml`` next to the ``.bin`` / ``.idx`` shards of one data source.

The YAML carries, in this order, ``name``, ``tokenizer_hash``, ``dtype`` (numpy name of the token type), ``shards`` (one
mapping per shard: ``prefix``, ``num_documents``, ``token_count``, ``bin_blake2b``, ``idx_blake2b``), ``filter_version``
and ``raw_jsonl_blake2b`` - the file format of the reference (src/pretrain/data/manifest.py:35-82), so manifests travel
between the two. The manifest is the one place mix weights and token counts are read from. File digests are blake2b-256,
the hash of the state digests, streamed in 1 MiB blocks.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field, fields
from functools import cached_property
from pathlib import Path

import yaml

_BLOCK = 1 << 20


def blake2b_file(path: str | Path, chunk_size: int = _BLOCK) -> str:
    digest = hashlib.blake2b(digest_size=32)
    buf = bytearray(chunk_size)
    view = memoryview(buf)
    with open(path, "rb", buffering=0) as f:
        while n := f.readinto(buf):
            digest.update(view[:n])
    return digest.hexdigest()


def _record(obj) -> dict:
    """A dataclass instance as a plain mapping in field order (the YAML key order)."""
    return {f.name: getattr(obj, f.name) for f in fields(obj)}


@dataclass
class ShardInfo:
    prefix: str                # path stem without .bin / .idx, relative to the manifest's directory unless absolute
    num_documents: int
    token_count: int
    bin_blake2b: str = ""      # empty = not recorded
    idx_blake2b: str = ""

    def files(self, base_dir: str | Path) -> list[tuple[Path, str]]:
        stem = Path(self.prefix)
        stem = stem if stem.is_absolute() else Path(base_dir) / stem
        return [(Path(str(stem) + ".bin"), self.bin_blake2b), (Path(str(stem) + ".idx"), self.idx_blake2b)]


@dataclass
class SourceManifest:
    name: str
    tokenizer_hash: str
    dtype: str
    shards: list[ShardInfo]
    filter_version: str = ""
    raw_jsonl_blake2b: dict[str, str] = field(default_factory=dict)

    # ---- totals (summed once; a manifest is not edited after it is built, `merged` / `from_dict` make new ones)
    @cached_property
    def _totals(self) -> tuple[int, int]:
        tokens = documents = 0
        for shard in self.shards:
            tokens += shard.token_count
            documents += shard.num_documents
        return tokens, documents

    @property
    def total_tokens(self) -> int:
        return self._totals[0]

    @property
    def total_documents(self) -> int:
        return self._totals[1]

    # ---- YAML
    def to_dict(self) -> dict:
        out = _record(self)
        out["shards"] = [_record(s) for s in self.shards]
        out["raw_jsonl_blake2b"] = dict(self.raw_jsonl_blake2b)
        return out

    @classmethod
    def from_dict(cls, data: dict) -> "SourceManifest":
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(data) - known)
        if unknown:
            raise ValueError("manifest has unknown keys %s" % unknown)
        body = dict(data)
        body["shards"] = [s if isinstance(s, ShardInfo) else ShardInfo(**s) for s in body.get("shards") or []]
        return cls(**body)

    def to_yaml(self) -> str:
        return yaml.safe_dump(self.to_dict(), sort_keys=False)

    @classmethod
    def from_yaml(cls, text: str) -> "SourceManifest":
        return cls.from_dict(yaml.safe_load(text))

    @classmethod
    def load(cls, path: str | Path) -> "SourceManifest":
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(yaml.safe_load(f))

    def save(self, path: str | Path) -> None:
        target = Path(path)
        target.parent.mkdir(parents=True, exist_ok=True)
        with open(target, "w", encoding="utf-8") as f:
            f.write(self.to_yaml())

    def hash(self) -> str:
        """sha256 of the YAML text: two manifests with the same content have the same hash."""
        return hashlib.sha256(self.to_yaml().encode("utf-8")).hexdigest()

    # ---- integrity
    def verify(self, base_dir: str | Path) -> list[str]:
        """Paths of shard files whose blake2b digest differs from the recorded one (unrecorded digests are skipped)."""
        return [str(p) for shard in self.shards for p, want in shard.files(base_dir) if want and blake2b_file(p) != want]
