"""Seed-generated synthetic corpora written as ordinary shards + manifest, so that synthetic runs go
through exactly the same stream, hashing and replay machinery as real data, and a replay can rebuild
the corpus from the seed alone (reference src/pretrain/cli/prepare_data.py:227-266)."""
from __future__ import annotations

from pathlib import Path

import numpy as np

from .indexed_dataset import IndexedDatasetWriter
from .manifest import ShardInfo, SourceManifest, blake2b_file


def write_uniform_source(out_dir: str | Path, name: str, vocab_size: int, seed: int, total_tokens: int, doc_len: tuple[int, int] = (64, 2048),
                         docs_per_shard: int = 4096, low_token: int = 1) -> SourceManifest:
    """Documents of uniform-random tokens in [low_token, vocab_size) (token 0 is left to the separator)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(np.array([seed, 0x5EED], dtype=np.uint64))
    shards, written, shard_id = [], 0, 0
    while written < total_tokens:
        prefix = "%s_%05d" % (name, shard_id)
        with IndexedDatasetWriter(out / prefix, np.uint32) as wtr:
            for _ in range(docs_per_shard):
                n = int(rng.integers(doc_len[0], doc_len[1] + 1))
                wtr.add_document(rng.integers(low_token, vocab_size, size=n, dtype=np.int64))
                written += n
                if written >= total_tokens:
                    break
            nd, nt = wtr.num_documents, wtr.token_count
        shards.append(ShardInfo(prefix, nd, nt, blake2b_file(str(out / prefix) + ".bin"), blake2b_file(str(out / prefix) + ".idx")))
        shard_id += 1
    man = SourceManifest(name=name, tokenizer_hash="synthetic-uniform-v%d" % vocab_size, dtype="uint32", shards=shards)
    man.save(out / "manifest.yaml")
    return man


def ensure_synthetic_sources(cfg, data_root: str | Path, tokens_needed: int) -> None:
    """Create every configured source that does not exist yet under ``data_root`` (deterministic in cfg.run.seed)."""
    for i, src in enumerate(cfg.data.sources):
        p = Path(src.path)
        p = p if p.is_absolute() else Path(data_root) / p
        if (p / "manifest.yaml").exists():
            continue
        share = cfg.data.normalised_weights()[i]
        write_uniform_source(p, src.name, cfg.model.vocab_size, cfg.run.seed * 1000 + i, int(tokens_needed * share * 1.25) + 4 * cfg.data.seq_len)
