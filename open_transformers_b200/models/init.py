"""Weight initialisation from ONE counter-based Philox stream.

Walking ``named_parameters()`` in module order, every parameter with >= 2 dims takes the next
``numel`` words of the stream keyed by ``seed`` and becomes ``std * z`` with z a standard normal
truncated to [-2, 2]; 1-D parameters are zero, norm gains one. The stream is sampled on the CPU
and the bytes are copied to the device, so the result is identical on every backend and for any
work split (reference src/pretrain/model/init.py:47-125).
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops.functional import trunc_normal_


def init_weights(model: nn.Module, seed: int | None, std: float | None = None) -> None:
    """``seed=None`` is the legacy path of single-process experiments: matrices come from torch's global generator (which
    ``parallel.env.set_seed`` offsets by rank, so ranks would differ) instead of the Philox stream; nothing that is hashed
    or replayed uses it. (reference src/pretrain/model/init.py:47-84)"""
    cfg = getattr(model, "cfg", None)
    if std is None:
        std = cfg.init.std if cfg is not None else 0.02
    offset = 0
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2 and seed is None:
                nn.init.trunc_normal_(p, std=std, a=-2 * std, b=2 * std)
            elif p.dim() >= 2:
                direct = p.device.type == "cpu" and p.dtype == torch.float32 and p.is_contiguous()
                buf = p.data if direct else torch.empty(p.shape, dtype=torch.float32)   # fp32 host parameters are filled in place
                trunc_normal_(buf, std, seed, offset)
                offset += p.numel()
                if not direct:
                    p.copy_(buf.to(p.dtype))
            elif name.endswith("norm.weight") or ".norm" in name or "norm_" in name or name.endswith("_norm.weight"):
                p.fill_(1.0)
            else:
                p.zero_()
        # the learned int8 step sizes are 1-D (zeroed above): derive them from the FINAL weights, last
        # (reference src/pretrain/model/init.py:150-199)
        from .modules.core import QuantLinear
        for m in model.modules():
            if isinstance(m, QuantLinear) and m.method == "lsq":
                m.weight_scale.copy_(m.lsq_optimal_scale(m.weight.detach().float()))


def init_weights_seeded(model: nn.Module, seed: int) -> None:
    """``init_weights`` with the model's configured spread: same seed, same bytes, on every device."""
    init_weights(model, seed)
