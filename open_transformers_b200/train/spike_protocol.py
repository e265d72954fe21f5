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
from collections import deque
from dataclasses import dataclass


class Halt(Exception):
    """Too many spikes in the window: stop the run and page a human."""


@dataclass
class SpikeProtocolState:
    skipped_steps: int = 0
    last_skip_step: int = -1
    halted: bool = False
    halt_reason: str = ""


class SpikeProtocol:
    def __init__(self, threshold: float, skips_in_window_to_halt: int, halt_window_steps: int, skip_steps_on_spike: int = 1,
                 start_step: int = 0):
        self.threshold = float(threshold)
        self.skips_in_window_to_halt = int(skips_in_window_to_halt)
        self.halt_window_steps = int(halt_window_steps)
        self.skip_steps_on_spike = max(1, int(skip_steps_on_spike))
        self.start_step = int(start_step)
        self._fresh: deque[int] = deque()
        self._cooldown = 0
        self.state = SpikeProtocolState()

    @classmethod
    def from_config(cls, spike_cfg) -> "SpikeProtocol":
        return cls(spike_cfg.grad_norm_threshold, spike_cfg.skips_in_window_to_halt, spike_cfg.halt_window_steps,
                   spike_cfg.skip_steps_on_spike, spike_cfg.start_step)

    def should_skip(self, grad_norm: float, loss: float, step: int = 0) -> bool:
        if not math.isfinite(loss) or not math.isfinite(grad_norm):
            return True
        if self._cooldown > 0:
            return True
        return step >= self.start_step and grad_norm > self.threshold

    def record_skip(self, step: int) -> None:
        self.state.skipped_steps += 1
        self.state.last_skip_step = step
        if self._cooldown > 0:          # a cool-down skip is not a new event
            self._cooldown -= 1
            return
        self._fresh.append(step)
        while self._fresh and self._fresh[0] < step - self.halt_window_steps:
            self._fresh.popleft()
        self._cooldown = self.skip_steps_on_spike - 1
        if len(self._fresh) >= self.skips_in_window_to_halt:
            self.state.halted = True
            self.state.halt_reason = "%d spikes within %d steps (threshold %g)" % (len(self._fresh), self.halt_window_steps, self.threshold)
            raise Halt(self.state.halt_reason)

    def state_dict(self) -> dict:
        return {"recent_skip_steps": list(self._fresh), "cooldown_remaining": self._cooldown, "skipped_steps": self.state.skipped_steps,
                "last_skip_step": self.state.last_skip_step, "halted": self.state.halted, "halt_reason": self.state.halt_reason}

    def load_state_dict(self, sd: dict) -> None:
        self._fresh = deque(int(s) for s in sd.get("recent_skip_steps", []))
        self._cooldown = int(sd.get("cooldown_remaining", 0))
        self.state = SpikeProtocolState(int(sd.get("skipped_steps", 0)), int(sd.get("last_skip_step", -1)), bool(sd.get("halted", False)),
                                        str(sd.get("halt_reason", "")))
