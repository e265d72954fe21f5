"""Token-clocked learning-rate schedules (tokens, not steps, are the clock, so a change of the
global batch size mid-run does not shift the curve). All arithmetic is Python double precision
and the result is hashed as part of ``param_groups``.

Shapes (reference src/pretrain/optim/schedules.py:28-107):
  cosine         linear warm-up, then half-cosine from peak to ``min_lr_frac * peak`` over the rest;
  wsd            warm-up, flat peak, linear decay from ``wsd_decay_start_frac * total`` to
                 ``wsd_decay_to_frac * peak``;
  linear_anneal  warm-up, flat peak until the ABSOLUTE token count ``anneal_start_tokens``, then
                 linear to ``min_lr_frac * peak`` at ``total`` (mid-training branch).
Warm-up length in tokens = ``warmup_steps`` x the warm-up phase's global batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass


def _clamp01(x: float) -> float:
    return 0.0 if x < 0.0 else (1.0 if x > 1.0 else x)


@dataclass(frozen=True)
class LRSchedule:
    kind: str
    peak: float
    end: float
    warmup_tokens: int
    total_tokens: int
    decay_start_frac: float = 0.0
    anneal_start_tokens: int = 0

    def __call__(self, consumed_tokens: int, total_tokens: int | None = None) -> float:
        total = self.total_tokens if total_tokens is None else total_tokens
        c = consumed_tokens
        if c < self.warmup_tokens:
            return self.peak * c / max(self.warmup_tokens, 1)
        if self.kind == "cosine":
            span = max(total - self.warmup_tokens, 1)
            t = _clamp01((c - self.warmup_tokens) / span)
            return self.end + 0.5 * (self.peak - self.end) * (1 + math.cos(math.pi * t))
        start = self.decay_start_frac * total if self.kind == "wsd" else max(self.anneal_start_tokens, self.warmup_tokens)
        if c < start:
            return self.peak
        t = _clamp01((c - start) / max(total - start, 1))
        return self.peak + (self.end - self.peak) * t


def _warmup_tokens(sched, train) -> int:
    return sched.warmup_steps * train.global_batch_tokens.warmup


def cosine_schedule(sched, train, optim) -> LRSchedule:
    return LRSchedule("cosine", optim.peak_lr, optim.peak_lr * sched.min_lr_frac, _warmup_tokens(sched, train), train.total_tokens)


def wsd_schedule(sched, train, optim) -> LRSchedule:
    return LRSchedule("wsd", optim.peak_lr, optim.peak_lr * sched.wsd_decay_to_frac, _warmup_tokens(sched, train), train.total_tokens,
                      decay_start_frac=sched.wsd_decay_start_frac)


def linear_anneal_schedule(sched, train, optim) -> LRSchedule:
    if train.total_tokens <= sched.anneal_start_tokens:
        raise ValueError("linear_anneal: train.total_tokens (%d) is absolute (pre-training + mid-training) and must exceed "
                         "schedule.anneal_start_tokens (%d)" % (train.total_tokens, sched.anneal_start_tokens))
    return LRSchedule("linear_anneal", optim.peak_lr, optim.peak_lr * sched.min_lr_frac, _warmup_tokens(sched, train), train.total_tokens,
                      anneal_start_tokens=sched.anneal_start_tokens)


SCHEDULES = {"cosine": cosine_schedule, "wsd": wsd_schedule, "linear_anneal": linear_anneal_schedule}


def build_schedule(sched, train, optim) -> LRSchedule:
    if sched.name not in SCHEDULES:
        raise ValueError("unknown schedule %r" % sched.name)
    return SCHEDULES[sched.name](sched, train, optim)


def rewarm_factor(consumed_tokens: int, anchor_tokens: int | None, rewarm_tokens: int) -> float:
    """Linear 0 -> 1 ramp over ``rewarm_tokens`` after a resume anchored at ``anchor_tokens``."""
    if not rewarm_tokens or anchor_tokens is None:
        return 1.0
    return _clamp01((consumed_tokens - anchor_tokens) / rewarm_tokens)


def schedule_lr(param_groups, lr: float) -> None:
    for g in param_groups:
        g["lr"] = float(lr)
