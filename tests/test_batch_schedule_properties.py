"""Properties of the global-batch schedule over random recipes: the step plans tile the window stream without gaps, the
token and window clocks agree, every micro-batch has exactly one owner and the owners' shares add up, a window maps back
to its (micro-batch, slot), and resuming the plan iterator at any step boundary continues the same sequence."""
import itertools
import types

import pytest
from hypothesis import given, settings, strategies as st

from open_transformers_b200.train.batch_schedule import (accum_for_rank, iter_step_plans, microbatch_indices_for_rank, microbatches_per_step,
                                                         owner_rank, window_position, windows_consumed_before)


def _train(mb, seq, warm, main, late, t1, t2):
    gbt = types.SimpleNamespace(warmup=warm, main=main, late=late)
    return types.SimpleNamespace(micro_batch_size=mb, seq_len=seq, global_batch_tokens=gbt, warmup_to_main_at_tokens=t1, main_to_late_at_tokens=t2)


recipes = st.builds(_train, st.integers(1, 4), st.sampled_from([32, 64, 96]), st.integers(64, 2000), st.integers(64, 4000), st.integers(64, 8000),
                    st.integers(0, 20000), st.integers(0, 60000))


@settings(max_examples=80, deadline=None)
@given(train=recipes, world=st.integers(1, 9), cut=st.integers(0, 30))
def test_plans_tile_the_stream_and_resume_anywhere(train, world, cut):
    plans = list(itertools.islice(iter_step_plans(0, 0, train), 40))
    tokens = windows = 0
    for i, p in enumerate(plans):
        assert p.step == i and p.consumed_tokens == tokens and p.base_window == windows
        assert p.microbatches == microbatches_per_step(tokens, train) >= 1
        per = train.micro_batch_size * train.seq_len
        target = (train.global_batch_tokens.warmup if tokens < train.warmup_to_main_at_tokens else
                  train.global_batch_tokens.main if tokens < train.main_to_late_at_tokens else train.global_batch_tokens.late)
        assert (p.microbatches - 1) * per < max(target, 1) <= p.microbatches * per or (target <= per and p.microbatches == 1)
        assert p.tokens_this_step == p.microbatches * per
        owners = [owner_rank(m, world_size=world) for m in range(p.microbatches)]
        assert sum(accum_for_rank(p.microbatches, world_size=world, rank=r) for r in range(world)) == p.microbatches
        for r in range(world):
            assert microbatch_indices_for_rank(p.microbatches, world_size=world, rank=r) == [m for m, o in enumerate(owners) if o == r]
        last = p.base_window + p.microbatches * train.micro_batch_size - 1
        assert window_position(p.base_window, p, micro_batch_size=train.micro_batch_size) == (0, 0)
        assert window_position(last, p, micro_batch_size=train.micro_batch_size) == (p.microbatches - 1, train.micro_batch_size - 1)
        with pytest.raises(ValueError):
            window_position(last + 1, p, micro_batch_size=train.micro_batch_size)
        tokens += p.tokens_this_step
        windows += p.microbatches * train.micro_batch_size
    at = plans[cut]
    assert windows_consumed_before(at.consumed_tokens, train) == at.base_window
    resumed = list(itertools.islice(iter_step_plans(at.consumed_tokens, at.base_window, train, start_step=at.step), 40 - cut))
    assert resumed == plans[cut:]
    if at.tokens_this_step > 1:
        with pytest.raises(ValueError):
            windows_consumed_before(at.consumed_tokens + 1, train)    # not a step boundary
