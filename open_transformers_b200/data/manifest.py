"""Per-source shard manifest (``manifest.yaml`` next to the shards) with blake2b-256 file digests
(reference src/pretrain/data/manifest.py:19-82)."""
from __future__ import annotations

import dataclasses
import hashlib
from pathlib import Path

import yaml


def blake2b_file(path: str | Path, chunk_size: int = 1 << 20) -> str:
    h = hashlib.blake2b(digest_size=32)
    with open(path, "rb") as f:
        while True:
            block = f.read(chunk_size)
            if not block:
                break
            h.update(block)
    return h.hexdigest()


@dataclasses.dataclass
class ShardInfo:
    prefix: str
    num_documents: int
    token_count: int
    bin_blake2b: str = ""
    idx_blake2b: str = ""


@dataclasses.dataclass
class SourceManifest:
    name: str
    tokenizer_hash: str
    dtype: str
    shards: list[ShardInfo]
    filter_version: str = ""
    raw_jsonl_blake2b: dict[str, str] = dataclasses.field(default_factory=dict)

    @property
    def total_tokens(self) -> int:
        return sum(s.token_count for s in self.shards)

    @property
    def total_documents(self) -> int:
        return sum(s.num_documents for s in self.shards)

    def to_yaml(self) -> str:
        return yaml.safe_dump(dataclasses.asdict(self), sort_keys=False)

    @classmethod
    def from_yaml(cls, text: str) -> "SourceManifest":
        d = yaml.safe_load(text)
        d["shards"] = [ShardInfo(**s) for s in d["shards"]]
        return cls(**d)

    @classmethod
    def load(cls, path: str | Path) -> "SourceManifest":
        return cls.from_yaml(Path(path).read_text(encoding="utf-8"))

    def save(self, path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(self.to_yaml(), encoding="utf-8")

    def hash(self) -> str:
        return hashlib.sha256(self.to_yaml().encode("utf-8")).hexdigest()

    def verify(self, base_dir: str | Path) -> list[str]:
        """Names of shard files whose digest does not match the manifest."""
        bad = []
        for s in self.shards:
            p = Path(s.prefix) if Path(s.prefix).is_absolute() else Path(base_dir) / s.prefix
            for ext, want in ((".bin", s.bin_blake2b), (".idx", s.idx_blake2b)):
                if want and blake2b_file(str(p) + ext) != want:
                    bad.append(str(p) + ext)
        return bad
