"""Building blocks of the decoder. Every module keeps an fp32 parameter (the master weight that
the optimizer and the state hash see) and, when the training engine installs one, a
compute-dtype view of the same weight plus a gradient slot (see ops/autograd.py). Parameter
names are the canonical hashed names and never change with wrapping or parallelism.
"""
from __future__ import annotations

import torch
from torch import nn

from ...ops import autograd as A
from ...ops import functional as K
from ..registry import ATTENTION, EMBEDDING, FFN, NORM, ROPE


class ParamMixin:
    """compute weight / gradient slot bookkeeping shared by the parametrised modules"""

    def _cw(self, name: str = "weight"):
        return getattr(self, "_compute_" + name, None)

    def _slot(self, name: str = "weight"):
        return getattr(self, "_slot_" + name, None)


class Linear(nn.Module, ParamMixin):
    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x, residual=None):
        w = self._cw()
        if w is None and x.dtype != self.weight.dtype:
            w = self.weight.to(x.dtype)
        return A.linear(x, self.weight, w, self._slot(), residual)


@NORM.register("rmsnorm_repop")
class RMSNorm(nn.Module, ParamMixin):
    """y = x * rsqrt(mean(x^2) + eps) * weight, fp32 inside; ``gain=False`` drops the weight."""

    def __init__(self, dim: int, eps: float = 1e-5, gain: bool = True):
        super().__init__()
        self.dim, self.eps = dim, eps
        if gain:
            self.weight = nn.Parameter(torch.ones(dim))
        else:
            self.register_parameter("weight", None)

    def forward(self, x):
        if self.weight is None:
            return A.rms_norm(x, None, eps=self.eps)
        w = self._cw()
        if w is None and x.dtype != self.weight.dtype:
            w = self.weight.to(x.dtype)
        return A.rms_norm(x, self.weight, w, self._slot(), self.eps)


@ROPE.register("rope_default")
class RoPE(nn.Module):
    """cos/sin tables [T, head_dim/2] in fp32, non-persistent; rotation is applied in fp32 inside
    the fused QK-norm/RoPE kernel with one rounding to the activation dtype."""

    def __init__(self, head_dim: int, max_seq_len: int, theta: float):
        super().__init__()
        self.head_dim, self.max_seq_len, self.theta = head_dim, max_seq_len, theta
        cos, sin = self._tables()
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def _tables(self):
        return K.rope_tables(self.max_seq_len, self.head_dim, self.theta, "cpu")

    def forward(self, seq_len: int):
        if self.rope_cos.dtype != torch.float32:  # a module-wide .to(bf16) must not touch the tables
            raise TypeError("RoPE tables must stay fp32")
        return self.rope_cos[:seq_len], self.rope_sin[:seq_len]


@ROPE.register("rope_yarn")
class RoPEYarn(RoPE):
    """NTK-by-parts (YaRN) frequency interpolation for long-context annealing: low-frequency
    dimensions are divided by ``factor``, high-frequency ones kept, with a linear ramp between.
    (reference src/pretrain/model/modules/rope.py:60-100)"""

    def __init__(self, head_dim, max_seq_len, theta, factor: float = 4.0, original_max: int = 4096,
                 beta_fast: float = 32.0, beta_slow: float = 1.0):
        self.factor, self.original_max, self.beta_fast, self.beta_slow = factor, original_max, beta_fast, beta_slow
        super().__init__(head_dim, max_seq_len, theta)

    def _tables(self):
        import math

        import numpy as np

        half = self.head_dim // 2
        j = np.arange(half, dtype=np.float64)
        inv = 1.0 / np.power(np.float64(self.theta), j / half)

        def corr(nrot):
            return self.head_dim * math.log(self.original_max / (nrot * 2 * math.pi)) / (2 * math.log(self.theta))

        lo, hi = max(math.floor(corr(self.beta_fast)), 0), min(math.ceil(corr(self.beta_slow)), half - 1)
        ramp = np.clip((j - lo) / max(hi - lo, 1e-3), 0.0, 1.0)
        inv = inv / self.factor * ramp + inv * (1.0 - ramp)
        pos = np.arange(self.max_seq_len, dtype=np.float64)[:, None] * inv[None, :]
        # numpy's double cos/sin are platform libm; the yarn variant is therefore CPU-built once and
        # shipped inside checkpoints' provenance rather than recomputed on other machines.
        return torch.from_numpy(np.cos(pos).astype(np.float32)), torch.from_numpy(np.sin(pos).astype(np.float32))


class _GQABase(nn.Module, ParamMixin):
    """Grouped-query attention: separate wq/wk/wv/wo parameters, one fused QKV GEMM at run time,
    optional QK RMSNorm over head_dim (with or without gain), interleaved-pair RoPE, causal or
    sliding-window flash attention, output projection fused with the residual add."""

    qk_norm_default = True

    def __init__(self, d_model, n_heads, n_kv_heads, head_dim, *, layer_idx=0, n_layers=1, swa_window=0,
                 swa_full_every=1, qk_norm=None, qk_norm_gain=True, eps=1e-5, attn_int8_pv=False):
        super().__init__()
        self.d_model, self.n_heads, self.n_kv_heads, self.head_dim = d_model, n_heads, n_kv_heads, head_dim
        self.eps = eps
        self.attn_int8_pv = attn_int8_pv
        full = (layer_idx % swa_full_every == swa_full_every - 1) or (layer_idx == n_layers - 1)
        self.window = 0 if (full or swa_window == 0) else swa_window
        self.wq = Linear(d_model, n_heads * head_dim)
        self.wk = Linear(d_model, n_kv_heads * head_dim)
        self.wv = Linear(d_model, n_kv_heads * head_dim)
        self.wo = Linear(n_heads * head_dim, d_model)
        self.qk_norm = self.qk_norm_default if qk_norm is None else qk_norm
        self.qk_norm_gain = bool(self.qk_norm and qk_norm_gain)
        if self.qk_norm_gain:
            self.q_norm = RMSNorm(head_dim, eps)
            self.k_norm = RMSNorm(head_dim, eps)

    def _qkv(self, x):
        fused = getattr(self, "_fused_qkv", None)
        if fused is not None:  # (master view, compute view, slot) spanning wq|wk|wv in the flat buffers
            return A.linear(x, fused[0], fused[1], fused[2])
        w = torch.cat([self.wq.weight, self.wk.weight, self.wv.weight], 0)
        return A.linear(x, w, w if w.dtype == x.dtype else w.to(x.dtype))

    def forward(self, x, cos, sin, residual=None):
        B, T, _ = x.shape
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self._qkv(x)
        if self.qk_norm_gain:
            q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
            q = self.q_norm(q.reshape(B, T, H, D)).reshape(B, T, H * D)
            k = self.k_norm(k.reshape(B, T, Hkv, D)).reshape(B, T, Hkv * D)
            qkv = torch.cat([q, k, v], -1)
            o = A.attention(qkv, cos, sin, H, Hkv, D, self.window, False, self.eps)
        else:
            o = A.attention(qkv, cos, sin, H, Hkv, D, self.window, self.qk_norm, self.eps)
        return self.wo(o, residual)


@ATTENTION.register("gqa_qknorm_repop")
class GQAQKNorm(_GQABase):
    qk_norm_default = True


@ATTENTION.register("gqa_plain_repop")
class GQAPlain(_GQABase):
    qk_norm_default = False

    def __init__(self, *a, **kw):
        kw["qk_norm"] = False
        super().__init__(*a, **kw)


@FFN.register("swiglu_repop")
class SwiGLU(nn.Module):
    """down( silu(gate) * up ) with gate and up produced by one GEMM (rows [0,F) = gate, [F,2F) = up)."""

    def __init__(self, d_model: int, intermediate: int):
        super().__init__()
        self.w_gate_up = Linear(d_model, 2 * intermediate)
        self.w_down = Linear(intermediate, d_model)

    def forward(self, x, residual=None):
        return self.w_down(A.swiglu(self.w_gate_up(x)), residual)


class Embedding(nn.Module, ParamMixin):
    def __init__(self, vocab: int, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim))

    def forward(self, ids, dtype=None):
        w = self._cw()
        if w is None and dtype is not None and dtype != self.weight.dtype:
            w = self.weight.to(dtype)
        return A.embedding(ids, self.weight, w, self._slot())


@EMBEDDING.register("untied_repop")
class UntiedEmbedding(nn.Module):
    """Input table and output projection with separate weights; the backward of the gather is
    the sorted, fixed-order segment sum (no atomics)."""

    def __init__(self, vocab_size: int, d_model: int):
        super().__init__()
        self.tok_embeddings = Embedding(vocab_size, d_model)
        self.output = Linear(d_model, vocab_size)

    def encode(self, ids, dtype=None):
        return self.tok_embeddings(ids, dtype)

    def project(self, hidden):
        return self.output(hidden)
