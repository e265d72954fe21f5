"""Spike handling: detect -> skip (with cool-down) -> halt.

A step is skipped (no optimizer update) when the loss or the pre-clip gradient norm is not finite,
when a cool-down from an earlier spike is still running, or - after ``start_step`` - when the
gradient norm exceeds ``threshold``. A fresh spike starts a cool-down of ``skip_steps_on_spike - 1``
further skipped steps. ``skips_in_window_to_halt`` fresh spikes within ``halt_window_steps`` steps
raise ``Halt``. The mutable part (cool-down counter, recent spike steps, totals) is checkpointed so
that a resume inside a cool-down or between two spikes behaves like the uninterrupted run
(reference src/pretrain/train/spike_protocol.py:62-131).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field


class Halt(Exception):
    """Too many spikes in the window: stop the run and page a human."""


@dataclass
class SpikeProtocolState:
    """Everything that changes during a run; ``asdict`` of it, under the key names of ``KEYS``, is ``spike_protocol.json``."""
    skipped_steps: int = 0
    last_skip_step: int = -1
    halted: bool = False
    halt_reason: str = ""
    cooldown: int = 0                                   # skips still owed to the last fresh spike
    fresh: list = field(default_factory=list)           # steps of the fresh spikes inside the halt window, ascending


# field -> key in the checkpoint file (the reference's names)
KEYS = {"fresh": "recent_skip_steps", "cooldown": "cooldown_remaining", "skipped_steps": "skipped_steps", "last_skip_step": "last_skip_step",
        "halted": "halted", "halt_reason": "halt_reason"}


class SpikeProtocol:
    def __init__(self, threshold: float, skips_in_window_to_halt: int, halt_window_steps: int, skip_steps_on_spike: int = 1,
                 start_step: int = 0):
        self.threshold, self.start_step = float(threshold), int(start_step)
        self.skips_in_window_to_halt, self.halt_window_steps = int(skips_in_window_to_halt), int(halt_window_steps)
        self.skip_steps_on_spike = max(1, int(skip_steps_on_spike))
        self.state = SpikeProtocolState()

    @classmethod
    def from_config(cls, spike_cfg) -> "SpikeProtocol":
        return cls(spike_cfg.grad_norm_threshold, spike_cfg.skips_in_window_to_halt, spike_cfg.halt_window_steps,
                   spike_cfg.skip_steps_on_spike, spike_cfg.start_step)

    def should_skip(self, grad_norm: float, loss: float, step: int = 0) -> bool:
        """Not finite: always (warm-up or not). Cool-down running: yes, whatever the norm says - and the caller still reports
        the skip, which is what counts the cool-down down. Otherwise the threshold, once ``start_step`` is reached."""
        if not (math.isfinite(loss) and math.isfinite(grad_norm)) or self.state.cooldown > 0:
            return True
        return step >= self.start_step and grad_norm > self.threshold

    def record_skip(self, step: int) -> None:
        st = self.state
        st.skipped_steps, st.last_skip_step = st.skipped_steps + 1, step
        if st.cooldown > 0:                 # part of an earlier event: not counted towards the halt
            st.cooldown -= 1
            return
        st.fresh = [s for s in st.fresh if s >= step - self.halt_window_steps] + [step]
        st.cooldown = self.skip_steps_on_spike - 1      # this call was the first of the skips
        if len(st.fresh) >= self.skips_in_window_to_halt:
            st.halted = True
            st.halt_reason = "%d spikes within %d steps (threshold %g)" % (len(st.fresh), self.halt_window_steps, self.threshold)
            raise Halt(st.halt_reason)

    def state_dict(self) -> dict:
        """The mutable state only (thresholds come from the configuration again on resume). Without it a resume just after a
        spike would step the optimizer in the middle of the cool-down, and two spikes on either side of a checkpoint
        would not add up to a halt."""
        return {key: (list(v) if isinstance(v, list) else v) for f, key in KEYS.items() for v in [getattr(self.state, f)]}

    def load_state_dict(self, sd: dict) -> None:
        blank = SpikeProtocolState()
        self.state = SpikeProtocolState(**{f: type(getattr(blank, f))(sd.get(key, getattr(blank, f))) for f, key in KEYS.items()})
        self.state.fresh = [int(s) for s in self.state.fresh]
