"""Held-out perplexity with a sliding window: each window of ``seq_len`` tokens is scored on its last
``stride`` positions (all of them for the first window), so every token is predicted with up to
``seq_len - stride`` tokens of context (reference src/pretrain/eval/perplexity.py)."""
from __future__ import annotations

import math

import torch

from ..ops import functional as K


@torch.no_grad()
def sliding_window_nll(model, tokens: torch.Tensor, seq_len: int, stride: int | None = None, device=None) -> tuple[float, int]:
    """Sum of negative log-likelihoods (nats) and number of scored tokens for a 1-D token tensor."""
    stride = stride or seq_len
    device = device or next(model.parameters()).device
    model.eval()
    n = tokens.numel()
    total, count, prev_end = 0.0, 0, 0
    for begin in range(0, max(n - 1, 1), stride):
        end = min(begin + seq_len, n - 1)
        ids = tokens[begin:end].unsqueeze(0).to(device)
        labels = tokens[begin + 1:end + 1].clone().unsqueeze(0)
        labels[:, : max(prev_end - begin, 0)] = -100      # already scored by the previous window
        logits = model(ids).logits
        l2 = logits.reshape(-1, logits.shape[-1]).contiguous()
        ce, _ = K.ce_zloss_(l2, labels.reshape(-1).to(device).contiguous(), 0.0, 1.0, write_grad=False)
        total += float(ce.double().sum())
        count += int((labels >= 0).sum())
        prev_end = end
        if end >= n - 1:
            break
    return total, count


def perplexity(model, tokens: torch.Tensor, seq_len: int, stride: int | None = None) -> float:
    nll, n = sliding_window_nll(model, tokens, seq_len, stride)
    return math.exp(nll / max(n, 1))
