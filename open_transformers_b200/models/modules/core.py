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

    # how a tensor-parallel group splits this layer: None (replicated compute), "col" (output features; ``tp_slices``
    # lists, per call, the (start, stop) ranges of one rank), "row" (inner dimension), "token" (token rows, full weight)
    tp_mode: str | None = None

    def tp_slices(self, st) -> list:
        """Output-feature ranges of every rank for a column-parallel layer (default: one contiguous block each)."""
        return [[st.split(self.out_features, r)] for r in range(st.size)]

    def forward(self, x, residual=None):
        w = self._cw()
        if w is None and x.dtype != self.weight.dtype:
            w = self.weight.to(x.dtype)
        st = A.tp()
        if st is not None and self.tp_mode is not None:
            wc = self.weight if w is None else w
            if self.tp_mode == "col":
                assert residual is None
                return A.tp_column_linear(x, self.weight, wc, self._slot(), self.tp_slices(st))
            if self.tp_mode == "row":
                return A.tp_row_linear(x, self.weight, wc, self._slot(), residual, [st.split(self.in_features, r) for r in range(st.size)])
            assert residual is None
            return A.tp_token_linear(x, self.weight, wc, self._slot())
        return A.linear(x, self.weight, w, self._slot(), residual)


class QuantLinear(Linear):
    """int8 quantisation-aware linear layer (W8A8). ``method``:

    * ``lsq``: learned per-output-channel step size ``weight_scale`` [out] (a parameter the optimizer sees; it is
      re-derived from the initial weights by ``init_weights`` and optionally re-pinned every N steps);
    * ``absmax``: step = max|w| / qmax per channel (``per_channel_w``) or per tensor, recomputed from the weights.

    ``qat_active`` is the warm-start switch: while false the layer is bit-identical to a plain ``Linear`` on the
    same weights; it is a pure function of (step, config) set by ``set_qat_active`` at the top of every step and
    never enters a checkpoint. (reference src/pretrain/model/modules/_linear.py:31-65,
    src/pretrain/model/modules/qat_warmstart.py:40-59)"""

    qat_active: bool = True

    def __init__(self, in_features, out_features, *, method="lsq", weight_bits=8, act_bits=8, per_channel_w=True, ste_bwd_hadamard=False):
        super().__init__(in_features, out_features)
        self.ste_bwd_hadamard = bool(ste_bwd_hadamard)  # both backward GEMMs as Hadamard-rotated int8 products
        self.method, self.weight_bits, self.act_bits, self.per_channel_w = method, weight_bits, act_bits, per_channel_w
        self.qmax_w, self.qmax_a = K.qmax_for_bits(weight_bits), K.qmax_for_bits(act_bits)
        if method == "lsq":
            self.weight_scale = nn.Parameter(torch.ones(out_features))
        self._qcache: dict = {}

    def lsq_optimal_scale(self, w: torch.Tensor) -> torch.Tensor:
        """2 mean|w_row| / sqrt(qmax), floored at 1e-6 (Esser et al.; reference src/pretrain/model/init.py:150-199)."""
        return K.row_stat(w.contiguous(), "mean_abs", 2.0 / (self.qmax_w ** 0.5), 1e-6)

    def _step(self, w):
        if self.method == "lsq":
            s = self._cw("weight_scale")
            s = self.weight_scale if s is None else s
            return s.detach().float().contiguous()
        if self.per_channel_w:
            return K.row_stat(w, "absmax", 1.0 / self.qmax_w, 1e-12)
        return (K.absmax(w) * (1.0 / self.qmax_w)).clamp_min(1e-12).expand(w.shape[0]).contiguous()

    def forward(self, x, residual=None, tp_mode=None):
        if not self.qat_active:
            return super().forward(x, residual)
        w = self._cw()
        if w is None:
            w = self.weight if x.dtype == self.weight.dtype else self.weight.to(x.dtype)
        w = w.detach()
        lsq = self.method == "lsq"
        st = A.tp()
        mode = tp_mode or self.tp_mode
        if st is not None and mode is not None:
            if self.ste_bwd_hadamard:
                raise NotImplementedError("the Hadamard int8 backward is not split over a tensor-parallel group")
            parts = self.tp_slices(st) if mode == "col" else [st.split(self.in_features, r) for r in range(st.size)]
            return A.tp_quant_linear(x, self.weight, w, self._slot(), self.weight_scale if lsq else None, self._step(w),
                                     self._slot("weight_scale") if lsq else None, residual, self.qmax_w, self.qmax_a, lsq, self._qcache,
                                     mode, parts)
        return A.quant_linear(x, self.weight, w, self._slot(), self.weight_scale if lsq else None, self._step(w),
                              self._slot("weight_scale") if lsq else None, residual, self.qmax_w, self.qmax_a, lsq, self._qcache, self.ste_bwd_hadamard)


def build_linear(in_features: int, out_features: int, qat=None, layer_idx: int = 0) -> Linear:
    """Plain or quantisation-aware linear layer, by the ``qat`` section of the model config; the first
    ``exempt_first_n_blocks`` blocks stay unquantised (reference src/pretrain/model/modules/_linear.py:31-65)."""
    if qat is None or not qat.enabled or layer_idx < qat.exempt_first_n_blocks:
        return Linear(in_features, out_features)
    return QuantLinear(in_features, out_features, method=qat.method, weight_bits=qat.weight_bits, act_bits=qat.act_bits,
                       per_channel_w=qat.per_channel_w, ste_bwd_hadamard=qat.ste_bwd_hadamard)


def set_qat_active(module: nn.Module, active: bool) -> int:
    """Flip the warm-start switch of every quantised layer under ``module``; returns how many were touched."""
    n = 0
    for m in module.modules():
        if isinstance(m, QuantLinear):
            m.qat_active = bool(active)
            n += 1
    return n


def refresh_lsq_weight_scales(module: nn.Module) -> int:
    """Re-pin every learned step size to the LSQ-optimal value of the CURRENT compute weights, writing both the
    fp32 parameter and its compute copy (reference repop.qat.lsq.refresh_lsq_weight_scales, called from
    src/pretrain/train/loop.py:1069-1084)."""
    n = 0
    with torch.no_grad():
        for m in module.modules():
            if isinstance(m, QuantLinear) and m.method == "lsq":
                w = m._cw()
                w = m.weight if w is None else w
                s = m.lsq_optimal_scale(w.detach())
                m.weight_scale.copy_(s)
                cs = m._cw("weight_scale")
                if cs is not None and cs.data_ptr() != m.weight_scale.data_ptr():
                    cs.copy_(s)
                n += 1
    return n


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

    def forward(self, x, tp_heads: int = 0):
        if self.weight is None:
            return A.rms_norm(x, None, eps=self.eps)
        w = self._cw()
        if w is None and x.dtype != self.weight.dtype:
            w = self.weight.to(x.dtype)
        return A.rms_norm(x, self.weight, w, self._slot(), self.eps, tp_heads)


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


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """The rotation written out on tensors: ``x`` [..., T, H, head_dim], tables [T, head_dim/2]; element pairs
    (2j, 2j+1) of every head turn by the angle of position t and frequency j. The training path applies the same rotation
    inside the fused QK-norm / RoPE kernel; this form serves tests and tools.
    (reference src/pretrain/model/modules/rope.py:103-125)"""
    even, odd = x[..., 0::2], x[..., 1::2]
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return torch.stack([even * c - odd * s, even * s + odd * c], -1).flatten(-2)


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
                 swa_full_every=1, qk_norm=None, qk_norm_gain=True, eps=1e-5, attn_int8_pv=False, qat=None):
        super().__init__()
        self.d_model, self.n_heads, self.n_kv_heads, self.head_dim = d_model, n_heads, n_kv_heads, head_dim
        self.eps = eps
        self.attn_int8_pv = attn_int8_pv
        full = (layer_idx % swa_full_every == swa_full_every - 1) or (layer_idx == n_layers - 1)
        self.window = 0 if (full or swa_window == 0) else swa_window
        self.wq = build_linear(d_model, n_heads * head_dim, qat, layer_idx)
        self.wk = build_linear(d_model, n_kv_heads * head_dim, qat, layer_idx)
        self.wv = build_linear(d_model, n_kv_heads * head_dim, qat, layer_idx)
        self.wo = build_linear(n_heads * head_dim, d_model, qat, layer_idx)
        self.wo.tp_mode = "row"   # heads are split over a tensor-parallel group; wq/wk/wv go through the fused weight
        self.qk_norm = self.qk_norm_default if qk_norm is None else qk_norm
        self.qk_norm_gain = bool(self.qk_norm and qk_norm_gain)
        if self.qk_norm_gain:
            self.q_norm = RMSNorm(head_dim, eps)
            self.k_norm = RMSNorm(head_dim, eps)

    def _int8_pv(self, qkv) -> bool:
        """``attn_int8_pv`` selects the int8 P V forward where the kernels exist (bf16 activations, head_dim 128);
        other shapes keep the float P V kernels and say so once."""
        if not self.attn_int8_pv:
            return False
        if K.int8_pv_supported(qkv.dtype, self.head_dim):
            return True
        if not getattr(_GQABase, "_warned_int8_pv", False):
            _GQABase._warned_int8_pv = True
            import logging
            logging.getLogger(__name__).warning("attn_int8_pv needs bf16 activations and head_dim 128 (got %s, %d): float P V kernels used",
                                                qkv.dtype, self.head_dim)
        return False

    def _qkv(self, x):
        if isinstance(self.wq, QuantLinear) and self.wq.qat_active:
            return torch.cat([self.wq(x), self.wk(x), self.wv(x)], -1)
        fused = getattr(self, "_fused_qkv", None)
        if fused is not None:  # (master view, compute view, slot) spanning wq|wk|wv in the flat buffers
            return A.linear(x, fused[0], fused[1], fused[2])
        w = torch.cat([self.wq.weight, self.wk.weight, self.wv.weight], 0)
        return A.linear(x, w, w if w.dtype == x.dtype else w.to(x.dtype))

    def _forward_tp(self, st, x, cos, sin, residual):
        """Tensor-parallel attention: ``x`` and ``residual`` are this rank's token rows [M/P, d]; the rank attends with
        H/P query heads and Hkv/P key/value heads over all tokens."""
        H, Hkv, D, P = self.n_heads, self.n_kv_heads, self.head_dim, st.size
        if H % P or Hkv % P:
            raise ValueError("%d query / %d key-value heads do not split over %d tensor-parallel ranks" % (H, Hkv, P))
        fused = getattr(self, "_fused_qkv", None)
        hq, hk = H * D // P, Hkv * D // P
        if isinstance(self.wq, QuantLinear) and self.wq.qat_active:
            # quantised projections keep their own step sizes: three column-parallel layers, this rank's heads of each
            qkv = torch.cat([self.wq(x, tp_mode="col"), self.wk(x, tp_mode="col"), self.wv(x, tp_mode="col")], -1)
        elif fused is None:
            raise NotImplementedError("tensor-parallel attention needs the fused QKV weight of the training engine")
        else:
            slices = [[(r * hq, (r + 1) * hq), (H * D + r * hk, H * D + (r + 1) * hk), ((H + Hkv) * D + r * hk, (H + Hkv) * D + (r + 1) * hk)]
                      for r in range(P)]
            qkv = A.tp_column_linear(x, fused[0], fused[1], fused[2], slices)
        B, T = st.batch_shape
        qk_norm = self.qk_norm
        if self.qk_norm_gain:  # the gains' gradients run over all heads: see RMSNormFn
            q, k, v = qkv.split([hq, hk, hk], -1)
            q = self.q_norm(q.reshape(B * T, H // P, D), tp_heads=H // P).reshape(B * T, hq)
            k = self.k_norm(k.reshape(B * T, Hkv // P, D), tp_heads=Hkv // P).reshape(B * T, hk)
            qkv, qk_norm = torch.cat([q, k, v], -1), False
        o = A.attention(qkv.view(B, T, -1), cos, sin, H // P, Hkv // P, D, self.window, qk_norm, self.eps, False)
        return self.wo(o.reshape(B * T, -1), residual)

    def forward(self, x, cos, sin, residual=None):
        st = A.tp()
        if st is not None:
            return self._forward_tp(st, x, cos, sin, residual)
        B, T, _ = x.shape
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self._qkv(x)
        if self.qk_norm_gain:
            q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
            q = self.q_norm(q.reshape(B, T, H, D)).reshape(B, T, H * D)
            k = self.k_norm(k.reshape(B, T, Hkv, D)).reshape(B, T, Hkv * D)
            qkv = torch.cat([q, k, v], -1)
            o = A.attention(qkv, cos, sin, H, Hkv, D, self.window, False, self.eps, self._int8_pv(qkv))
        else:
            o = A.attention(qkv, cos, sin, H, Hkv, D, self.window, self.qk_norm, self.eps, self._int8_pv(qkv))
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

    def __init__(self, d_model: int, intermediate: int, qat=None, layer_idx: int = 0):
        super().__init__()
        self.intermediate = intermediate
        self.w_gate_up = build_linear(d_model, 2 * intermediate, qat, layer_idx)
        self.w_down = build_linear(intermediate, d_model, qat, layer_idx)
        # tensor parallel: rank r takes gate columns and up columns [r F/P, (r+1) F/P) and the matching inner slice of w_down
        self.w_gate_up.tp_mode, self.w_down.tp_mode = "col", "row"
        F = intermediate
        self.w_gate_up.tp_slices = lambda st: [[st.split(F, r), tuple(F + v for v in st.split(F, r))] for r in range(st.size)]

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
        self.output.tp_mode = "token"  # the head keeps the whole vocabulary and works on the rank's token rows

    def encode(self, ids, dtype=None):
        return self.tok_embeddings(ids, dtype)

    def project(self, hidden):
        return self.output(hidden)
