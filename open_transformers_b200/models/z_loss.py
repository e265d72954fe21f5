"""Stand-alone z-loss: ``coeff * mean_n(lse_n^2)`` over the (batch, token) rows of a logits tensor, with the
explicit gradient ``(2 coeff / N) * lse_n * softmax[n, v]``.

The training step uses the fused CE + z-loss kernel (``fused_loss.py``); this module is the separate entry point for
callers that want the auxiliary term, its row statistics or its gradient on their own (evaluation, the frugal audit
path, tests). Every row is reduced by the same fixed-order kernel as the fused loss, so ``row_lse`` and the fused
loss agree bit for bit, and a row's result does not depend on how many rows are passed
(reference src/pretrain/model/z_loss.py:52-140).
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from ..ops import functional as K

Z_LOSS_GRAD_CHUNK_ROWS = 2048
_LN2 = 0.6931471805599453


def row_lse(logits: torch.Tensor) -> torch.Tensor:
    """Natural-log log-sum-exp of every row of ``logits`` [..., V] as fp32 [...]; the logits are left untouched."""
    l2 = logits.reshape(-1, logits.shape[-1]).contiguous().clone()
    labels = torch.zeros(l2.shape[0], dtype=torch.long, device=l2.device)
    _, lse = K.ce_zloss_(l2, labels, 0.0, 1.0, write_grad=False)
    return lse.view(logits.shape[:-1])


def z_loss_grad(logits: torch.Tensor, coeff: float, grad_z: torch.Tensor | float = 1.0, chunk_rows: int = Z_LOSS_GRAD_CHUNK_ROWS) -> torch.Tensor:
    """``d z_loss / d logits`` in the dtype of ``logits``, evaluated ``chunk_rows`` rows at a time (the per-row
    result does not depend on the chunking). N is the total row count."""
    l2 = logits.reshape(-1, logits.shape[-1])
    n = l2.shape[0]
    out = torch.empty_like(l2)
    gz = float(grad_z)
    for r0 in range(0, n, chunk_rows):
        chunk = l2[r0:r0 + chunk_rows].float()
        lse = row_lse(chunk)
        soft = torch.exp(chunk - lse[:, None])
        out[r0:r0 + chunk_rows] = (soft * (lse * (2.0 * coeff * gz / n))[:, None]).to(out.dtype)
    return out.view(logits.shape)


class _ZLossFn(Function):
    @staticmethod
    def forward(ctx, logits, coeff):
        lse = row_lse(logits).reshape(-1)
        ctx.save_for_backward(logits)
        ctx.coeff = coeff
        return (K.det_sum(lse, True, 1.0 / lse.numel()) * coeff).reshape(())

    @staticmethod
    def backward(ctx, gz):
        (logits,) = ctx.saved_tensors
        return z_loss_grad(logits, ctx.coeff, gz), None


def compute_z_loss(logits: torch.Tensor, cfg_or_coeff) -> torch.Tensor:
    """Scalar z-loss of ``logits``; ``cfg_or_coeff`` is a ``ZLossConfig`` (``enabled``, ``coeff``) or a float.
    A disabled config (or coeff 0) returns an exact zero that carries no gradient."""
    coeff = float(cfg_or_coeff) if isinstance(cfg_or_coeff, (int, float)) else (float(cfg_or_coeff.coeff) if cfg_or_coeff.enabled else 0.0)
    if coeff == 0.0:
        return torch.zeros((), dtype=torch.float32, device=logits.device)
    return _ZLossFn.apply(logits, coeff)


def compute_z_loss_inert(logits: torch.Tensor, cfg_or_coeff) -> torch.Tensor:
    """The value of the z-loss without its gradient: the regime of runs made before the term had a backward pass, kept so
    that such a run's logged loss can be recomputed. (reference src/pretrain/model/z_loss.py:132-146)"""
    with torch.no_grad():
        return compute_z_loss(logits.detach(), cfg_or_coeff)
