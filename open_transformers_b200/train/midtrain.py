"""Guards for a mid-training (linear-anneal) branch: the branch must start exactly at the checkpoint
it was planned from, with its optimizer state, and the absolute token budget must lie beyond it
(reference src/pretrain/train/midtrain.py:51-107)."""
from __future__ import annotations


class MidtrainConfigError(ValueError):
    pass


def check_linear_anneal_resume(cfg, resume_consumed_tokens: int | None) -> None:
    sched = cfg.schedule
    if sched.name != "linear_anneal":
        return
    start = sched.anneal_start_tokens
    if start == 0:
        return  # cold linear-anneal run
    if resume_consumed_tokens is None:
        raise MidtrainConfigError("schedule.anneal_start_tokens=%d needs --resume-from a checkpoint at that token count" % start)
    if resume_consumed_tokens != start:
        raise MidtrainConfigError("mid-training branch point mismatch: checkpoint has consumed_tokens=%d but schedule.anneal_start_tokens=%d"
                                  % (resume_consumed_tokens, start))
    if cfg.train.resume_reset_optimizer:
        raise MidtrainConfigError("mid-training continues the optimizer state: train.resume_reset_optimizer must be false")
    if cfg.train.total_tokens <= start:
        raise MidtrainConfigError("train.total_tokens (%d) is absolute and must exceed the branch point (%d)" % (cfg.train.total_tokens, start))
    if sched.warmup_steps * cfg.train.global_batch_tokens.warmup > start:
        raise MidtrainConfigError("warm-up would extend past the branch point")
