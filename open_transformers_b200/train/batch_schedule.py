"""Global-batch schedule and the canonical per-step layout (no world-size term anywhere).

Phases by consumed tokens: warm-up batch until ``warmup_to_main_at_tokens``, main batch until
``main_to_late_at_tokens``, late batch after. A step consumes M = ceil(target / (mb * seq)) micro-batches,
i.e. M * mb consecutive windows of the global stream; micro-batch m belongs to data-parallel rank
m % V (reference src/pretrain/train/batch_schedule.py:31-209).
"""
from __future__ import annotations

import dataclasses


def current_global_batch_tokens(consumed_tokens: int, train) -> int:
    if consumed_tokens < train.warmup_to_main_at_tokens:
        return train.global_batch_tokens.warmup
    if consumed_tokens < train.main_to_late_at_tokens:
        return train.global_batch_tokens.main
    return train.global_batch_tokens.late


def microbatches_per_step(consumed_tokens: int, train) -> int:
    per = train.micro_batch_size * train.seq_len
    return max(1, -(-current_global_batch_tokens(consumed_tokens, train) // per))


def windows_per_step(consumed_tokens: int, train) -> int:
    return microbatches_per_step(consumed_tokens, train) * train.micro_batch_size


def canonical_tokens_per_step(consumed_tokens: int, train) -> int:
    return windows_per_step(consumed_tokens, train) * train.seq_len


def grad_accum_steps(consumed_tokens: int, train, dp_world_size: int) -> int:
    """Legacy per-rank accumulation count: ceil(target / (mb * seq * world))."""
    per = train.micro_batch_size * train.seq_len * max(dp_world_size, 1)
    return max(1, -(-current_global_batch_tokens(consumed_tokens, train) // per))


def tokens_per_optimizer_step(consumed_tokens: int, train, *, dp_world_size: int) -> int:
    """Tokens one optimizer step consumes under the legacy per-rank accumulation rule (the canonical stream uses
    ``canonical_tokens_per_step``)."""
    return grad_accum_steps(consumed_tokens, train, dp_world_size) * train.micro_batch_size * train.seq_len * max(dp_world_size, 1)


def owner_rank(microbatch: int, *, world_size: int) -> int:
    return microbatch % max(world_size, 1)


def accum_for_rank(total_microbatches: int, *, world_size: int, rank: int) -> int:
    if not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    return len(range(rank, total_microbatches, world_size))


def microbatch_indices_for_rank(total_microbatches: int, *, world_size: int, rank: int) -> list[int]:
    return list(range(rank, total_microbatches, world_size))


@dataclasses.dataclass(frozen=True)
class StepPlan:
    step: int
    consumed_tokens: int   # before the step
    base_window: int       # index of the step's first window in the global stream
    microbatches: int
    tokens_this_step: int


def window_position(global_window: int, plan: StepPlan, *, micro_batch_size: int) -> tuple[int, int]:
    rel = global_window - plan.base_window
    if not 0 <= rel < plan.microbatches * micro_batch_size:
        raise ValueError("window %d is not part of step %d" % (global_window, plan.step))
    return divmod(rel, micro_batch_size)


def iter_step_plans(consumed_tokens: int, windows_emitted: int, train, *, start_step: int = 0):
    step = start_step
    while True:
        m = microbatches_per_step(consumed_tokens, train)
        tokens = m * train.micro_batch_size * train.seq_len
        yield StepPlan(step, consumed_tokens, windows_emitted, m, tokens)
        consumed_tokens += tokens
        windows_emitted += m * train.micro_batch_size
        step += 1


def default_interval_end(step: int, consumed_tokens: int, train) -> int:
    """The step at which the checkpoint interval that starts at (``step``, ``consumed_tokens``) ends: ``ckpt_every_steps``
    further on, or - when the recipe clocks checkpoints by tokens - the first step that crosses the next multiple of
    ``ckpt_every_tokens`` (or exhausts ``total_tokens``). The replay's default target and the span whose data is fetched."""
    if train.ckpt_every_steps == 0 and train.ckpt_every_tokens > 0:
        every, c, end = train.ckpt_every_tokens, consumed_tokens, step
        for plan in iter_step_plans(consumed_tokens, 0, train, start_step=step):
            end += 1
            c += plan.tokens_this_step
            if c // every > plan.consumed_tokens // every or c >= train.total_tokens:
                break
        return end
    return step + max(train.ckpt_every_steps, 1)


def windows_consumed_before(consumed_tokens: int, train) -> int:
    """Windows emitted by a run from token 0 up to ``consumed_tokens`` (must land on a step boundary)."""
    c = w = 0
    for plan in iter_step_plans(0, 0, train):
        if c >= consumed_tokens:
            break
        c += plan.tokens_this_step
        w += plan.microbatches * train.micro_batch_size
    if c != consumed_tokens:
        raise ValueError("consumed_tokens=%d is not a step boundary of this schedule" % consumed_tokens)
    return w
