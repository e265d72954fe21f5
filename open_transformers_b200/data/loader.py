"""Loaders: resolve configured sources into manifests + per-document mixing probabilities and build
the canonical per-process view. Batches are ``{"input_ids": w[:, :-1], "labels": w[:, 1:]}`` int64,
pinned when CUDA is present (reference src/pretrain/data/loader.py:37-187)."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from .global_stream import GlobalStream, GlobalStreamState, ShardedWindowView
from .manifest import SourceManifest
from .mix_sampler import MixSampler


def collate(windows: np.ndarray, pin: bool = False) -> dict[str, torch.Tensor]:
    t = torch.from_numpy(np.ascontiguousarray(windows, dtype=np.int64))
    batch = {"input_ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous()}
    if pin and torch.cuda.is_available():
        batch = {k: v.pin_memory() for k, v in batch.items()}
    return batch


def resolve_sources(data_cfg, data_root: str | None = None):
    """manifests, directories and DOCUMENT-draw probabilities. When the configured weights are token shares,
    a source with longer documents is drawn proportionally less often: p_i ~ share_i / mean_doc_len_i."""
    manifests, dirs = [], []
    for src in data_cfg.sources:
        p = Path(src.path)
        if data_root and not p.is_absolute():
            p = Path(data_root) / p
        manifests.append(SourceManifest.load(p / "manifest.yaml"))
        dirs.append(str(p))
    weights = data_cfg.normalised_weights()
    if data_cfg.weights_are_token_shares:
        mean_len = [m.total_tokens / max(m.total_documents, 1) for m in manifests]
        if any(l <= 0 for l in mean_len):
            raise ValueError("token-share weights need non-empty sources")
        raw = [w / l for w, l in zip(weights, mean_len)]
        weights = [r / sum(raw) for r in raw]
    return manifests, dirs, weights


def build_global_loader(cfg, ranks, world_size: int, state: GlobalStreamState | None = None, consumed_tokens: int = 0,
                        start_step: int = 0, data_root: str | None = None, index_only: bool = False, seed: int | None = None) -> ShardedWindowView:
    """``index_only``: a view that walks document lengths only (manifest + .idx, no .bin): for the step -> document map and
    the shard fetcher. ``seed``: the run's recorded seed where it is not the configuration's."""
    manifests, dirs, weights = resolve_sources(cfg.data, data_root)
    return ShardedWindowView(manifests, dirs, weights, cfg.data.seq_len, cfg.run.seed if seed is None else seed, cfg.train, ranks, world_size,
                             eos_id=cfg.data.document_separator_id, state=state, consumed_tokens=consumed_tokens, start_step=start_step,
                             index_only=index_only)


def build_global_stream(cfg, state: GlobalStreamState | None = None, data_root: str | None = None) -> GlobalStream:
    manifests, dirs, weights = resolve_sources(cfg.data, data_root)
    return GlobalStream(manifests, dirs, weights, cfg.data.seq_len, cfg.run.seed, cfg.data.document_separator_id, state)


def build_loader(cfg, rank: int, world_size: int, state=None, data_root: str | None = None) -> MixSampler:
    """Legacy topology-dependent loader (DDP runs)."""
    manifests, dirs, weights = resolve_sources(cfg.data, data_root)
    return MixSampler(manifests, dirs, weights, cfg.data.seq_len, cfg.run.seed, rank, world_size, cfg.data.document_separator_id, state)
