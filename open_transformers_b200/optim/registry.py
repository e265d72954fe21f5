"""Optimizer by config name (reference src/pretrain/optim/registry.py:13-27)."""
from __future__ import annotations


def build_optimizer(named_params, optim_cfg):
    name = optim_cfg.name
    if name in ("adamw", "adamw_repop"):
        from .adamw import build_adamw

        return build_adamw(named_params, optim_cfg)
    if name == "muon_hybrid":
        from .muon import MuonWithAuxAdamW

        return MuonWithAuxAdamW(named_params, optim_cfg)
    raise ValueError("unknown optimizer %r" % name)
