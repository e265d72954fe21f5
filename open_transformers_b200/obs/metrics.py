"""Metrics: model FLOPs, MFU, JSONL logger, timers."""
from __future__ import annotations

import contextlib
import json
import time
from pathlib import Path

B200_BF16_DENSE_PEAK = 2.25e15  # nominal dense bf16 FLOP/s of one B200


def tokens_per_sec(tokens: int, elapsed_s: float) -> float:
    return tokens / max(elapsed_s, 1e-9)


def transformer_flops_per_token(n_layers: int, d_model: int, seq_len: int, vocab_size: int) -> float:
    """Forward + backward FLOPs per token: 72 L d^2 (dense blocks) + 12 L s d (attention) + 6 V d (head)
    (reference src/pretrain/obs/metrics.py:23-47)."""
    return 72.0 * n_layers * d_model ** 2 + 12.0 * n_layers * seq_len * d_model + 6.0 * vocab_size * d_model


def hardware_flops_per_token(m, seq_len: int) -> float:
    """Forward + backward FLOPs per token that the kernels actually execute for a ``ModelConfig``: 6 FLOPs per matrix
    weight (GQA projections, fused gate/up, down, vocabulary head) plus, per layer, 12 d FLOPs per (query, visible key)
    pair - a query sees on average (T + 1) / 2 keys under the full causal mask and fewer than ``swa_window`` under the
    sliding one. The reference's formula above counts every layer as dense T x T attention and square projections; for the
    OPEN-1B shape it gives 11.24 GFLOP per token against 8.54 here."""
    d, hd = m.d_model, m.head_dim
    weights = m.n_layers * (d * m.n_heads * hd * 2 + d * m.n_kv_heads * hd * 2 + 3 * d * m.ffn_intermediate) + m.vocab_size * d
    full_keys = (seq_len + 1) / 2.0
    w = min(int(getattr(m, "swa_window", 0) or 0), seq_len)
    window_keys = (w * (w + 1) / 2.0 + (seq_len - w) * w) / seq_len if w else full_keys
    every = max(int(getattr(m, "swa_full_every", 1) or 1), 1)
    attn = 0.0
    for layer in range(m.n_layers):
        is_full = w == 0 or layer % every == every - 1 or layer == m.n_layers - 1
        attn += 12.0 * (m.n_heads * hd) * (full_keys if is_full else window_keys)
    return 6.0 * weights + attn


def count_parameters(m) -> int:
    """Parameter count of the decoder described by a ``ModelConfig`` (untied embedding and head, GQA projections, fused
    gate/up, two block norms, final norm; optional embedding norm and QK-norm gains)."""
    d, hd = m.d_model, m.head_dim
    attn = d * (m.n_heads * hd) * 2 + d * (m.n_kv_heads * hd) * 2
    qk = 2 * hd if (getattr(m, "qk_norm", False) and getattr(m, "qk_norm_gain", False)) else 0
    block = attn + 3 * d * m.ffn_intermediate + 2 * d + qk
    return 2 * m.vocab_size * d + m.n_layers * block + d + (d if getattr(m, "emb_norm", False) else 0)


def mfu(tokens_per_sec_per_gpu: float, flops_per_token: float, peak_flops: float = B200_BF16_DENSE_PEAK) -> float:
    return tokens_per_sec_per_gpu * flops_per_token / peak_flops


class MetricsLogger:
    """Rank-0 JSONL writer (flushed every ``flush_every`` rows and on close) with an optional W&B mirror."""

    def __init__(self, path: str | Path | None, wandb_run=None, flush_every: int = 100, enabled: bool = True):
        self.enabled = enabled and path is not None
        self.wandb = wandb_run
        self._n, self._every = 0, flush_every
        self._f = None
        if self.enabled:
            Path(path).parent.mkdir(parents=True, exist_ok=True)
            self._f = open(path, "a", encoding="utf-8")

    def log(self, row: dict, step: int | None = None) -> None:
        if self._f is not None:
            self._f.write(json.dumps(row, sort_keys=True, default=str) + "\n")
            self._n += 1
            if self._n % self._every == 0:
                self._f.flush()
        if self.wandb is not None:
            self.wandb.log(row, step=step)

    def close(self) -> None:
        if self._f is not None:
            self._f.flush()
            self._f.close()
            self._f = None
        if self.wandb is not None and hasattr(self.wandb, "finish"):
            self.wandb.finish()


@contextlib.contextmanager
def time_section(sink: dict, key: str):
    t0 = time.perf_counter()
    try:
        yield
    finally:
        sink[key] = sink.get(key, 0.0) + (time.perf_counter() - t0) * 1e3
