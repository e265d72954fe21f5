"""Controls for the learnable QK-norm gains: clamp the gains to a ceiling, and freeze the query gains for
the first steps by zeroing their gradient. Both are no-ops at their default (0) settings and for gain-free
models (reference src/pretrain/train/qk_gain_control.py:48-68)."""
from __future__ import annotations

import torch


def _gains(model, which: str):
    for name, p in model.named_parameters():
        if name.endswith("%s_norm.weight" % which):
            yield name, p


@torch.no_grad()
def clamp_qk_gains(model, max_gain: float) -> int:
    if max_gain <= 0:
        return 0
    n = 0
    for which in ("q", "k"):
        for _, p in _gains(model, which):
            p.clamp_(min=-max_gain, max=max_gain)  # symmetric, as the reference's clamp_(-cap, cap)
            n += 1
    # the compute-dtype copies that the forward pass reads (installed by the training engine) follow on every rank
    for mod in model.modules():
        cw = getattr(mod, "_compute_weight", None)
        if cw is not None and type(mod).__name__ == "RMSNorm" and any(mod is getattr(parent, a, None)
                                                                       for parent in model.modules() for a in ("q_norm", "k_norm")):
            if cw.data_ptr() != mod.weight.data_ptr():
                cw.clamp_(min=-max_gain, max=max_gain)
    return n


@torch.no_grad()
def zero_q_gain_grads(named_grads: dict, step: int, freeze_until_step: int) -> int:
    if freeze_until_step <= 0 or step >= freeze_until_step:
        return 0
    n = 0
    for name, g in named_grads.items():
        if name.endswith("q_norm.weight") and g is not None:
            g.zero_()
            n += 1
    return n
