"""Loss entry points: fused cross-entropy + z-loss over full logits, and the streaming head
variant that never materialises the [tokens, vocab] logits."""
from __future__ import annotations

import torch

from ..ops import autograd as A
from ..ops import functional as K

Z_LOSS_GRAD_CHUNK_ROWS = 2048


def fused_ce_z_loss(logits: torch.Tensor, labels: torch.Tensor, z_coeff: float, grad_scale: float = 1.0):
    """Returns (mean CE, z_coeff * mean lse^2). See ops.autograd.FusedCEZLossFn."""
    return A.fused_ce_z_loss(logits, labels, z_coeff, grad_scale)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Plain mean CE without gradient side effects (evaluation helper)."""
    l2 = logits.reshape(-1, logits.shape[-1]).contiguous().clone()
    ce, _ = K.ce_zloss_(l2, labels.reshape(-1).contiguous(), 0.0, 1.0, write_grad=False)
    n = int((labels.reshape(-1) >= 0).sum().item())
    return K.det_sum(ce, False, 1.0 / max(n, 1)).reshape(())


def streaming_head_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, z_coeff: float,
                        panel_rows: int = 2048, grad_scale: float = 1.0, slot=None):
    """Vocabulary head + loss in row panels: for each panel of ``panel_rows`` tokens the logits are
    produced, reduced to their loss rows, turned into gradients in place and immediately consumed by
    the two gradient GEMMs, so only one panel of logits exists at a time. dW accumulates over panels
    in ascending panel order with the fp32 accumulate epilogue, i.e. one long ascending-row chain per
    element, equal to the unstreamed weight gradient of the exact family
    (reference src/pretrain/model/streaming_head_loss.py:15-118).

    ``slot``: a gradient slot of the training engine (``ops.autograd.GradSlot``); the weight gradient then continues the
    chain already in ``slot.buf`` (or starts it, when this is the slot's first writer of the step) exactly as the
    unstreamed layer's accumulate epilogue does, and no separate dW is allocated.

    Returns (ce, z, d_hidden, d_weight[fp32])."""
    h2 = hidden.reshape(-1, hidden.shape[-1]).contiguous()
    lab = labels.reshape(-1).contiguous()
    n = h2.shape[0]
    inv_n = 1.0 / n
    ce_rows = torch.empty(n, dtype=torch.float32, device=h2.device)
    lse_rows = torch.empty(n, dtype=torch.float32, device=h2.device)
    dh = torch.empty_like(h2)
    store_first = False
    if slot is not None and slot.buf is not None:
        dW, store_first = slot.buf, slot.take()
    else:
        dW = torch.zeros(weight.shape, dtype=torch.float32, device=h2.device)
    for r0 in range(0, n, panel_rows):
        r1 = min(n, r0 + panel_rows)
        logits = K.gemm(h2[r0:r1], weight)
        ce, lse = K.ce_zloss_(logits, lab[r0:r1], z_coeff, inv_n * grad_scale, write_grad=True)
        ce_rows[r0:r1] = ce
        lse_rows[r0:r1] = lse
        K.gemm(logits, weight, b_mn=True, out=dh[r0:r1])
        K.gemm(logits, h2[r0:r1], a_mn=True, b_mn=True, out=dW, epi=K.EPI_STORE_F32 if (store_first and r0 == 0) else K.EPI_ACC_F32)
    ce = K.det_sum(ce_rows, False, inv_n).reshape(())
    z = (K.det_sum(lse_rows, True, inv_n) * z_coeff).reshape(())
    return ce, z, dh.view(hidden.shape), dW
