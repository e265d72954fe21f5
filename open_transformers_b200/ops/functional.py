"""Device-dispatching wrappers over the native kernels.

Every function takes torch tensors and runs the sm_100a kernel when they live on a CUDA device
or the bit-exact C++ twin when they live on the CPU. There is no PyTorch fallback: a missing
native library is an error. Activations are bf16 (tensor-core family) or fp32 (exact family).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import native as _native
from .native import D as _D, F, I, L, P, check, cpu_lib, cuda_lib, is_bf16, stream_ptr

_status_words: dict[int, torch.Tensor] = {}

EPI_STORE, EPI_STORE_F32, EPI_ACC_F32, EPI_RESIDUAL = 0, 1, 2, 3
NORM_SLAB = 8  # rows per dgamma slab (csrc/cuda/elementwise.cu)


def _status(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status_words[idx]


def kernel_status(device=None) -> int:
    """Non-zero if a bounded in-kernel wait ever gave up on this device (sync point)."""
    device = torch.device(device or "cuda")
    return int(_status(device)[0].item())


def _ld(t: torch.Tensor) -> int:
    """Leading dimension (row pitch in elements) of a 2-D operand. A dimension of size 1 may carry any stride (PyTorch
    calls such a tensor contiguous whatever it says), so it is ignored."""
    assert t.dim() == 2 and (t.stride(1) == 1 or t.shape[1] == 1), "operand must be a 2-D tensor with unit inner stride"
    if t.shape[0] == 1 and t.stride(0) < t.shape[1]:
        return t.shape[1]
    return t.stride(0)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         epi: int = EPI_STORE, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``C[M,N] = op(A) op(B)^T``. ``a``: [M,K] (or [K,M] when ``a_mn``), ``b``: [N,K] (or [K,N] when ``b_mn``).

    ``epi``: 0 store in the operand dtype, 1 store fp32, 2 accumulate into fp32 ``out``, 3 store
    ``acc + residual`` in the operand dtype. Summation order: ascending k, never split."""
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, "inner dimensions differ: %s vs %s" % (tuple(a.shape), tuple(b.shape))
    assert a.dtype == b.dtype and a.device == b.device
    bf = is_bf16(a)
    out_dtype = a.dtype if epi in (EPI_STORE, EPI_RESIDUAL) else torch.float32
    if out is None:
        assert epi != EPI_ACC_F32, "accumulating epilogue needs an output tensor"
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.dtype == out_dtype and tuple(out.shape) == (M, N)
    if epi == EPI_RESIDUAL:
        assert residual is not None and residual.dtype == a.dtype and tuple(residual.shape) == (M, N)
    ldr = _ld(residual) if residual is not None else 0
    if a.is_cuda:
        lib = cuda_lib()
        if bf:
            check(lib.otb_gemm_bf16(P(a), P(b), P(out), P(residual), I(M), I(N), I(K), L(_ld(a)), L(_ld(b)), L(_ld(out)),
                                    L(ldr), I(a_mn), I(b_mn), I(epi), P(_status(a.device)), I(0), stream_ptr()),
                  "gemm_bf16" if _native._timing is None else "gemm_bf16 %dx%dx%d %s%s epi%d" % (M, N, K, "tn"[a_mn], "tn"[b_mn], epi))
        else:
            check(lib.otb_gemm_f32(P(a), P(b), P(out), P(residual), I(M), I(N), I(K), L(_ld(a)), L(_ld(b)), L(_ld(out)),
                                   L(ldr), I(a_mn), I(b_mn), I(epi), stream_ptr()), "gemm_f32")
    else:
        check(cpu_lib().otb_cpu_gemm(P(a), P(b), P(out), P(residual), I(M), I(N), I(K), L(_ld(a)), L(_ld(b)), L(_ld(out)),
                                     L(ldr), I(a_mn), I(b_mn), I(epi), I(bf), I(bf)), "cpu_gemm")
    return out


# ------------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor | None, eps: float):
    rows, Dm = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    inv_d = 1.0 / Dm
    if x.is_cuda:
        check(cuda_lib().otb_rmsnorm_fwd(P(x), P(w), P(y), P(rstd), L(rows), I(Dm), F(inv_d), F(eps), I(is_bf16(x)), stream_ptr()), "rmsnorm_fwd")
    else:
        check(cpu_lib().otb_cpu_rmsnorm_fwd(P(x), P(w), P(y), P(rstd), L(rows), I(Dm), F(inv_d), F(eps), I(is_bf16(x))), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, w, rstd, need_dgamma: bool):
    rows, Dm = x.shape
    dx = torch.empty_like(x)
    lib = cuda_lib() if x.is_cuda else cpu_lib()
    slabs = (rows + NORM_SLAB - 1) // NORM_SLAB
    part = torch.empty((slabs, Dm), dtype=torch.float32, device=x.device) if need_dgamma else None
    inv_d = 1.0 / Dm
    if x.is_cuda:
        check(lib.otb_rmsnorm_bwd(P(dy), P(x), P(w), P(rstd), P(dx), P(part), L(rows), I(Dm), F(inv_d), I(is_bf16(x)), stream_ptr()), "rmsnorm_bwd")
    else:
        check(lib.otb_cpu_rmsnorm_bwd(P(dy), P(x), P(w), P(rstd), P(dx), P(part), L(rows), I(Dm), F(inv_d), I(is_bf16(x))), "rmsnorm_bwd")
    return dx, (part[0] if need_dgamma else None)


# ------------------------------------------------------------------ QK-norm + RoPE, attention
def qknorm_rope_fwd(qkv, cos, sin, heads: int, D: int, seq_len: int, do_norm: bool, eps: float):
    rows = qkv.shape[0]
    out = torch.empty((rows, heads * D), dtype=qkv.dtype, device=qkv.device)
    rstd = torch.empty(rows * heads if do_norm else 1, dtype=torch.float32, device=qkv.device)
    args = (P(qkv), L(_ld(qkv)), P(out), L(_ld(out)), P(rstd), P(cos), P(sin), L(rows), I(heads), I(D), I(seq_len), I(do_norm),
            F(1.0 / D), F(eps), I(is_bf16(qkv)))
    if qkv.is_cuda:
        check(cuda_lib().otb_qknorm_rope_fwd(*args, stream_ptr()), "qknorm_rope_fwd")
    else:
        check(cpu_lib().otb_cpu_qknorm_rope_fwd(*args), "qknorm_rope_fwd")
    return out, rstd


def qknorm_rope_bwd(dout, qkv, rstd, din, cos, sin, heads: int, D: int, seq_len: int, do_norm: bool):
    rows = qkv.shape[0]
    args = (P(dout), L(_ld(dout)), P(qkv), L(_ld(qkv)), P(rstd), P(din), L(_ld(din)), P(cos), P(sin), L(rows), I(heads), I(D),
            I(seq_len), I(do_norm), F(1.0 / D), I(is_bf16(qkv)))
    if qkv.is_cuda:
        check(cuda_lib().otb_qknorm_rope_bwd(*args, stream_ptr()), "qknorm_rope_bwd")
    else:
        check(cpu_lib().otb_cpu_qknorm_rope_bwd(*args), "qknorm_rope_bwd")
    return din


def int8_pv_supported(dtype: torch.dtype, D: int) -> bool:
    """The int8 P V kernels take bf16 activations and 128-wide heads (one 128-byte value row per key)."""
    return dtype == torch.bfloat16 and D == 128


def attn_fwd(qk, qkv, B: int, T: int, H: int, Hkv: int, D: int, window: int, int8_pv: bool = False):
    """qk: [B*T, (H+Hkv)*D] rotated queries+keys; qkv: [B*T, (H+2Hkv)*D] (values read from it).
    Returns O [B*T, H*D] and the row statistic lse [B,H,T] (log2 domain). ``int8_pv``: P V on the int8 tensor
    cores with per-block value quantisation (reference int8pv_causal_flash_attention, attention_repop.py:52)."""
    O = torch.empty((B * T, H * D), dtype=qk.dtype, device=qk.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=qk.device)
    scale = 1.0 / math.sqrt(D)
    if int8_pv:
        if not int8_pv_supported(qk.dtype, D):
            raise ValueError("int8 P V attention needs bf16 activations and head_dim 128 (got %s, %d)" % (qk.dtype, D))
        if qk.is_cuda:
            vq = torch.empty((B * T, Hkv * D), dtype=torch.int8, device=qk.device)
            vstep = torch.empty((B, Hkv, (T + 127) // 128), dtype=torch.float32, device=qk.device)
            check(cuda_lib().otb_attn_fwd_i8pv(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), P(vq), P(vstep), I(B), I(T),
                                               I(H), I(Hkv), I(D), I(window), F(scale), P(_status(qk.device)), stream_ptr()), "attn_fwd_i8pv")
        else:
            check(cpu_lib().otb_cpu_attn_fwd_i8pv(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv),
                                                  I(D), I(window), F(scale)), "cpu_attn_fwd_i8pv")
        return O, lse
    if qk.is_cuda:
        lib = cuda_lib()
        if is_bf16(qk):
            check(lib.otb_attn_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv), I(D),
                                   I(window), F(scale), P(_status(qk.device)), stream_ptr()),
                  "attn_fwd" if _native._timing is None else "attn_fwd w%d" % window)
        else:
            check(lib.otb_attn_f32_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv),
                                       I(D), I(window), F(scale), stream_ptr()), "attn_f32_fwd")
    else:
        check(cpu_lib().otb_cpu_attn_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv),
                                         I(D), I(window), F(scale), I(is_bf16(qk))), "cpu_attn_fwd")
    return O, lse


def attn_bwd(qk, qkv, O, dO, lse, dqk, dqkv, B: int, T: int, H: int, Hkv: int, D: int, window: int):
    """Writes dQ|dK into ``dqk`` and dV into the value columns of ``dqkv``."""
    delta = torch.empty((3, B, H, T), dtype=torch.float32, device=qk.device)  # delta, and the kernels' negated copies of lse / delta
    scale = 1.0 / math.sqrt(D)
    common = (P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(dO), L(_ld(dO)), P(lse), P(delta), P(dqk), L(_ld(dqk)),
              P(dqkv), L(_ld(dqkv)), I(B), I(T), I(H), I(Hkv), I(D), I(window), F(scale))
    if qk.is_cuda:
        lib = cuda_lib()
        if is_bf16(qk):
            check(lib.otb_attn_bwd(*common, P(_status(qk.device)), stream_ptr()),
                  "attn_bwd" if _native._timing is None else "attn_bwd w%d" % window)
        else:
            check(lib.otb_attn_f32_bwd(*common, stream_ptr()), "attn_f32_bwd")
    else:
        check(cpu_lib().otb_cpu_attn_bwd(*common, I(is_bf16(qk))), "cpu_attn_bwd")


# ------------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    rows, F2 = gu.shape
    h = torch.empty((rows, F2 // 2), dtype=gu.dtype, device=gu.device)
    if gu.is_cuda:
        check(cuda_lib().otb_swiglu_fwd(P(gu), P(h), L(rows), I(F2 // 2), I(is_bf16(gu)), stream_ptr()), "swiglu_fwd")
    else:
        check(cpu_lib().otb_cpu_swiglu_fwd(P(gu), P(h), L(rows), I(F2 // 2), I(is_bf16(gu))), "swiglu_fwd")
    return h


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor) -> torch.Tensor:
    rows, F2 = gu.shape
    dgu = torch.empty_like(gu)
    if gu.is_cuda:
        check(cuda_lib().otb_swiglu_bwd(P(gu), P(dh), P(dgu), L(rows), I(F2 // 2), I(is_bf16(gu)), stream_ptr()), "swiglu_bwd")
    else:
        check(cpu_lib().otb_cpu_swiglu_bwd(P(gu), P(dh), P(dgu), L(rows), I(F2 // 2), I(is_bf16(gu))), "swiglu_bwd")
    return dgu


# ---------------------------------------------------------------------------------- loss
def ce_zloss_(logits: torch.Tensor, labels: torch.Tensor, z_coeff: float, grad_scale: float, write_grad: bool = True):
    """Per-row CE and lse; when ``write_grad`` the logits are overwritten by d loss/d logits."""
    rows, V = logits.shape
    ce = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    two_z = 2.0 * z_coeff
    if logits.is_cuda:
        check(cuda_lib().otb_ce_zloss(P(logits), P(labels), P(ce), P(lse), L(rows), I(V), F(two_z), F(grad_scale), I(write_grad),
                                      I(is_bf16(logits)), stream_ptr()), "ce_zloss")
    else:
        check(cpu_lib().otb_cpu_ce_zloss(P(logits), P(labels), P(ce), P(lse), L(rows), I(V), F(two_z), F(grad_scale), I(write_grad),
                                         I(is_bf16(logits))), "ce_zloss")
    return ce, lse


def det_sum(x: torch.Tensor, squares: bool = False, post_scale: float = 1.0) -> torch.Tensor:
    """Canonical sum (or sum of squares) of a flat fp32 tensor, times ``post_scale``; 1-element tensor."""
    x = x.reshape(-1)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    if x.is_cuda:
        check(cuda_lib().otb_det_sum(P(x), L(x.numel()), I(squares), F(post_scale), P(out), stream_ptr()), "det_sum")
    else:
        check(cpu_lib().otb_cpu_det_sum(P(x), L(x.numel()), I(squares), F(post_scale), P(out)), "det_sum")
    return out


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    ids = ids.reshape(-1).contiguous()
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    if table.is_cuda:
        check(cuda_lib().otb_embedding_fwd(P(ids), P(table), P(out), L(ids.numel()), I(table.shape[1]), I(is_bf16(table)), stream_ptr()), "embedding_fwd")
    else:
        check(cpu_lib().otb_cpu_embedding_fwd(P(ids), P(table), P(out), L(ids.numel()), I(table.shape[1]), I(is_bf16(table))), "embedding_fwd")
    return out


def embedding_bwd(dy: torch.Tensor, ids: torch.Tensor, dW: torch.Tensor, accumulate: bool) -> None:
    """dW[id] (+)= sum of dy rows with that id, in ascending token position (stable sort, no atomics)."""
    ids = ids.reshape(-1)
    sorted_ids, order = torch.sort(ids, stable=True)
    sorted_ids, order, n = sorted_ids.contiguous(), order.contiguous(), ids.numel()
    if dy.is_cuda:
        check(cuda_lib().otb_embedding_bwd(P(dy), P(sorted_ids), P(order), L(n), P(dW), I(dW.shape[1]), I(accumulate), I(is_bf16(dy)),
                                           stream_ptr()), "embedding_bwd")
    else:
        check(cpu_lib().otb_cpu_embedding_bwd(P(dy), P(sorted_ids), P(order), L(n), P(dW), I(dW.shape[1]), I(accumulate), I(is_bf16(dy))),
              "embedding_bwd")


# --------------------------------------------------------------------------- RoPE tables
_rope_cache: dict = {}


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [seq_len, head_dim/2] fp32. Always computed by the CPU routine (double precision,
    deterministic operations only) and copied, so every device holds the same bytes."""
    key = (seq_len, head_dim, float(theta))
    if key not in _rope_cache:
        half = head_dim // 2
        cos = torch.empty((seq_len, half), dtype=torch.float32, device="cpu")  # explicit: a caller may build the model under
        sin = torch.empty((seq_len, half), dtype=torch.float32, device="cpu")  # a ``torch.device("meta")`` context
        cpu_lib().otb_cpu_rope_tables(P(cos), P(sin), I(seq_len), I(half), _D(theta))
        _rope_cache[key] = (cos, sin)
    cos, sin = _rope_cache[key]
    return cos.to(device), sin.to(device)


def trunc_normal_(out: torch.Tensor, std: float, seed: int, offset: int) -> None:
    """Fill a CPU fp32 tensor from the Philox stream (element i <- stream word offset+i)."""
    assert out.device.type == "cpu" and out.dtype == torch.float32 and out.is_contiguous()
    cpu_lib().otb_cpu_trunc_normal(P(out), L(out.numel()), F(std), ctypes.c_uint64(seed), ctypes.c_uint64(offset))


# ------------------------------------------------------------------------ int8 QAT (W8A8)
def qmax_for_bits(bits: int) -> int:
    """Largest magnitude of the symmetric signed grid: 127 for 8 bits (reference repop.qat.functional._qmax_for_bits,
    used at src/pretrain/model/init.py:168)."""
    if not 2 <= bits <= 8:
        raise ValueError("quantisation width must be 2..8 bits, got %d" % bits)
    return (1 << (bits - 1)) - 1


weight_epoch: int | None = None  # set (and bumped at every weight change) by the training engine; None = never cache


def absmax(x: torch.Tensor) -> torch.Tensor:
    """max |x| as a 1-element fp32 tensor (order-free, identical on every backend)."""
    x = x.reshape(-1)
    assert x.is_contiguous()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    if x.is_cuda:
        lib = cuda_lib()
        scratch = torch.empty(lib.otb_absmax_scratch_floats(), dtype=torch.float32, device=x.device)
        check(lib.otb_absmax(P(x), L(x.numel()), I(is_bf16(x)), P(scratch), P(out), stream_ptr()), "absmax")
    else:
        check(cpu_lib().otb_cpu_absmax(P(x), L(x.numel()), I(is_bf16(x)), P(out)), "absmax")
    return out


def quant_act(x: torch.Tensor, qmax: int):
    """Per-tensor symmetric quantisation: step = max|x| / qmax, q = clamp(rint(x / step)). Returns (q int8, step[1])."""
    assert x.is_contiguous()
    am = absmax(x)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    step = torch.empty(1, dtype=torch.float32, device=x.device)
    if x.is_cuda:
        check(cuda_lib().otb_quant_act(P(x), L(x.numel()), I(is_bf16(x)), P(am), I(qmax), P(q), P(step), stream_ptr()), "quant_act")
    else:
        check(cpu_lib().otb_cpu_quant_act(P(x), L(x.numel()), I(is_bf16(x)), P(am), I(qmax), P(q), P(step)), "quant_act")
    return q, step


def quant_weight(w: torch.Tensor, s: torch.Tensor, qmax: int, hat_dtype: torch.dtype | None = None):
    """Per-output-channel quantisation of ``w`` [N,K] by the step sizes ``s`` [N] (fp32): q = clamp(rint(w / s)).
    Returns (q int8 [N,K], w_hat = q * s in ``hat_dtype`` or None)."""
    N, Kd = w.shape
    assert w.is_contiguous() and s.dtype == torch.float32 and s.numel() == N and s.is_contiguous()
    q = torch.empty((N, Kd), dtype=torch.int8, device=w.device)
    hat = torch.empty((N, Kd), dtype=hat_dtype, device=w.device) if hat_dtype is not None else None
    hd = 0 if hat is None else is_bf16(hat)
    if w.is_cuda:
        check(cuda_lib().otb_quant_weight(P(w), P(s), L(N), I(Kd), I(is_bf16(w)), I(qmax), P(q), P(hat), I(hd), stream_ptr()), "quant_weight")
    else:
        check(cpu_lib().otb_cpu_quant_weight(P(w), P(s), L(N), I(Kd), I(is_bf16(w)), I(qmax), P(q), P(hat), I(hd)), "quant_weight")
    return q, hat


def gemm_i8(aq: torch.Tensor, bq: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor, out_dtype: torch.dtype,
            residual: torch.Tensor | None = None) -> torch.Tensor:
    """``C = float(A_q B_q^T) * (sa * sb[n]) (+ residual)``: int8 [M,K] x int8 [N,K], exact int32 accumulation
    (tcgen05 kind::i8 on the GPU), one rounding at the dequantisation."""
    M, Kd = aq.shape
    N, Kb = bq.shape
    assert Kd == Kb and aq.dtype == torch.int8 and bq.dtype == torch.int8
    assert sa.dtype == torch.float32 and sb.dtype == torch.float32 and sb.numel() == N
    out = torch.empty((M, N), dtype=out_dtype, device=aq.device)
    bf = is_bf16(out)
    epi = EPI_RESIDUAL if residual is not None else (EPI_STORE if bf else EPI_STORE_F32)
    if residual is not None:
        assert residual.dtype == out_dtype and tuple(residual.shape) == (M, N)
    ldr = _ld(residual) if residual is not None else 0
    if aq.is_cuda:
        late_add = residual is not None and not bf  # exact family: one IEEE add after the fp32 store, same bits as the twin
        if late_add:
            epi = EPI_STORE_F32
        check(cuda_lib().otb_gemm_i8(P(aq), P(bq), P(out), P(None if late_add else residual), I(M), I(N), I(Kd), L(_ld(aq)), L(_ld(bq)),
                                     L(_ld(out)), L(ldr), P(sa), P(sb), I(epi), P(_status(aq.device)), I(0), stream_ptr()), "gemm_i8")
        if late_add:
            out.add_(residual)
    else:
        check(cpu_lib().otb_cpu_gemm_i8(P(aq), P(bq), P(out), P(residual), I(M), I(N), I(Kd), L(_ld(aq)), L(_ld(bq)), L(_ld(out)), L(ldr),
                                        P(sa), P(sb), I(3 if residual is not None else 0), I(bf)), "gemm_i8")
    return out


def lsq_bwd_(G: torch.Tensor, w: torch.Tensor, s: torch.Tensor, ga: torch.Tensor | None, qmax: int, gs: float,
             dW: torch.Tensor, ds: torch.Tensor | None) -> None:
    """Straight-through backward of the learned step size, accumulating into ``dW`` [N,K] and ``ds`` [N] (fp32):
    ``dW += inside ? G*ga : 0``, ``ds += gs * sum_k G*ga * (inside ? rint(t)-t : sign(t) qmax)`` with t = w/s."""
    N, Kd = w.shape
    assert G.dtype == torch.float32 and G.is_contiguous() and dW.dtype == torch.float32 and dW.is_contiguous()
    learn = ds is not None
    if w.is_cuda:
        check(cuda_lib().otb_lsq_bwd(P(G), P(w), P(s), P(ga), L(N), I(Kd), I(is_bf16(w)), I(qmax), F(gs), P(dW), P(ds), I(learn), stream_ptr()), "lsq_bwd")
    else:
        check(cpu_lib().otb_cpu_lsq_bwd(P(G), P(w), P(s), P(ga), L(N), I(Kd), I(is_bf16(w)), I(qmax), F(gs), P(dW), P(ds), I(learn)), "lsq_bwd")


def row_stat(w: torch.Tensor, mode: str, c: float, floor: float) -> torch.Tensor:
    """Per-row statistic of ``w`` [N,K] as fp32 [N]: ``mean_abs``: max(c * mean_k|w|, floor); ``absmax``: max(c * max_k|w|, floor)."""
    N, Kd = w.shape
    assert w.is_contiguous()
    s = torch.empty(N, dtype=torch.float32, device=w.device)
    m = {"mean_abs": 0, "absmax": 1}[mode]
    if w.is_cuda:
        check(cuda_lib().otb_row_stat(P(w), L(N), I(Kd), I(is_bf16(w)), I(m), F(c), F(floor), P(s), stream_ptr()), "row_stat")
    else:
        check(cpu_lib().otb_cpu_row_stat(P(w), L(N), I(Kd), I(is_bf16(w)), I(m), F(c), F(floor), P(s)), "row_stat")
    return s


def i8_widen(q: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(q.shape, dtype=dtype, device=q.device)
    assert q.is_contiguous() and q.dtype == torch.int8
    if q.is_cuda:
        check(cuda_lib().otb_i8_widen(P(q), P(out), L(q.numel()), I(is_bf16(out)), stream_ptr()), "i8_widen")
    else:
        check(cpu_lib().otb_cpu_i8_widen(P(q), P(out), L(q.numel()), I(is_bf16(out))), "i8_widen")
    return out


HADAMARD_BLOCK = 128


def fwht_blocks(x: torch.Tensor, block: int = HADAMARD_BLOCK) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard transform of every aligned ``block`` of the last dimension of an fp32 matrix
    (H_block x_block, entries +-1). log2(block) butterfly stages of one correctly rounded add and one subtract per pair,
    in a fixed order, so the result is the same on every device; H H^T = block * I."""
    assert x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] % block == 0 and block & (block - 1) == 0
    R, C = x.shape
    y = x
    h = 1
    while h < block:
        y = y.reshape(R, C // (2 * h), 2, h)
        a, b = y[:, :, 0, :], y[:, :, 1, :]
        y = torch.stack((a + b, a - b), dim=2)
        h *= 2
    return y.reshape(R, C)


def quant_rows(x: torch.Tensor, qmax: int):
    """Per-row symmetric int8 quantisation of an fp32 / bf16 matrix: step_r = max(max_k |x_rk| / qmax, tiny); returns
    (q int8, step fp32 [rows])."""
    x = x.contiguous()
    step = row_stat(x, "absmax", 1.0 / qmax, 1e-30)
    q, _ = quant_weight(x, step, qmax)
    return q, step


def ste_matmul_hadamard(a: torch.Tensor, b: torch.Tensor, qmax: int = 127) -> torch.Tensor:
    """``a b^T`` ([R1, C] x [R2, C] -> fp32 [R1, R2]) on the int8 tensor cores: both operands are rotated by the block
    Hadamard transform along the contraction index (which cancels in the product and spreads outliers over the block),
    quantised per row to int8, multiplied exactly in int32 and dequantised in fp32:
    ``(float(acc) * sb[n]) * sa[m] * (1 / block)``. The contraction length must be a multiple of the block.
    (reference role: repop `_ste_matmul_hadamard` / bfr_hadamard_int8_gemm, docs/MODEL_OP_DTYPE_TRACE.md:104,113-116)"""
    ha, hb = fwht_blocks(a.float().contiguous()), fwht_blocks(b.float().contiguous())
    aq, sa = quant_rows(ha, qmax)
    bq, sb = quant_rows(hb, qmax)
    one = torch.ones(1, dtype=torch.float32, device=a.device)
    acc = gemm_i8(aq, bq, one, sb, torch.float32)
    return (acc * sa[:, None]) * (1.0 / HADAMARD_BLOCK)
