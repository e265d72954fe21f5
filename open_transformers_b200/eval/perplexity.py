"""Held-out perplexity with a sliding window: each window of ``seq_len`` tokens is scored on its last
``stride`` positions (all of them for the first window), so every token is predicted with up to
``seq_len - stride`` tokens of context (reference src/pretrain/eval/perplexity.py)."""
from __future__ import annotations

import math

import torch

from ..ops import functional as K


@torch.no_grad()
def sliding_window_nll(model, tokens: torch.Tensor, seq_len: int, stride: int | None = None, device=None,
                       batch_windows: int = 1) -> tuple[float, int]:
    """Sum of negative log-likelihoods (nats) and number of scored tokens for a 1-D token tensor. ``batch_windows``
    windows of equal length share one forward pass; the per-window sums stay on the device until the end (one host
    synchronisation per call, not per window)."""
    stride = stride or seq_len
    device = device or next(model.parameters()).device
    model.eval()
    n = tokens.numel()
    windows, prev_end = [], 0
    for begin in range(0, max(n - 1, 1), stride):
        end = min(begin + seq_len, n - 1)
        windows.append((begin, end, max(prev_end - begin, 0)))   # the first ``skip`` labels were scored by the previous window
        prev_end = end
        if end >= n - 1:
            break
    total = torch.zeros((), dtype=torch.float64, device=device)
    count = 0
    i = 0
    while i < len(windows):
        length = windows[i][1] - windows[i][0]
        group = [windows[i]]
        while len(group) < max(1, batch_windows) and i + len(group) < len(windows) and \
                windows[i + len(group)][1] - windows[i + len(group)][0] == length:
            group.append(windows[i + len(group)])
        i += len(group)
        ids = torch.stack([tokens[b:e] for b, e, _ in group]).to(device)
        labels = torch.stack([tokens[b + 1:e + 1] for b, e, _ in group]).clone()
        for row, (_, _, skip) in enumerate(group):
            labels[row, :skip] = -100
        logits = model(ids).logits
        l2 = logits.reshape(-1, logits.shape[-1]).contiguous()
        ce, _ = K.ce_zloss_(l2, labels.reshape(-1).to(device).contiguous(), 0.0, 1.0, write_grad=False)
        total += ce.double().sum()
        count += int((labels >= 0).sum())
    return float(total), count


def perplexity(model, tokens: torch.Tensor, seq_len: int, stride: int | None = None, batch_windows: int = 1) -> float:
    nll, n = sliding_window_nll(model, tokens, seq_len, stride, batch_windows=batch_windows)
    return math.exp(nll / max(n, 1))


def compute_perplexity(model, held_out_prefix, seq_len: int, device=None, micro_batch_size: int = 1, max_tokens: int | None = None) -> float:
    """Perplexity of a held-out ``.bin/.idx`` shard: its documents joined in order, scored in windows of ``seq_len``
    (``micro_batch_size`` windows per forward pass). (entry point of the reference's src/pretrain/eval/perplexity.py:22)"""
    import numpy as np

    from ..data.indexed_dataset import IndexedDatasetReader

    r = IndexedDatasetReader(held_out_prefix)
    toks = np.concatenate([np.asarray(r.document(i), dtype=np.int64) for i in range(len(r))])
    if max_tokens:
        toks = toks[:max_tokens]
    return perplexity(model, torch.from_numpy(toks), seq_len, None, micro_batch_size)

