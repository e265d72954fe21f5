"""Device-dispatching wrappers over the native kernels.

Every function takes torch tensors and runs the sm_100a kernel when they live on a CUDA device
or the bit-exact C++ twin when they live on the CPU. There is no PyTorch fallback: a missing
native library is an error. Activations are bf16 (tensor-core family) or fp32 (exact family).
"""
from __future__ import annotations

import ctypes
import math

import torch

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
    assert t.dim() == 2 and t.stride(1) == 1, "operand must be a 2-D tensor with unit inner stride"
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
                                    L(ldr), I(a_mn), I(b_mn), I(epi), P(_status(a.device)), I(0), stream_ptr()), "gemm_bf16")
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


def attn_fwd(qk, qkv, B: int, T: int, H: int, Hkv: int, D: int, window: int):
    """qk: [B*T, (H+Hkv)*D] rotated queries+keys; qkv: [B*T, (H+2Hkv)*D] (values read from it).
    Returns O [B*T, H*D] and the row statistic lse [B,H,T] (log2 domain)."""
    O = torch.empty((B * T, H * D), dtype=qk.dtype, device=qk.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=qk.device)
    scale = 1.0 / math.sqrt(D)
    if qk.is_cuda:
        lib = cuda_lib()
        if is_bf16(qk):
            check(lib.otb_attn_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv), I(D),
                                   I(window), F(scale), P(_status(qk.device)), stream_ptr()), "attn_fwd")
        else:
            check(lib.otb_attn_f32_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv),
                                       I(D), I(window), F(scale), stream_ptr()), "attn_f32_fwd")
    else:
        check(cpu_lib().otb_cpu_attn_fwd(P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(lse), I(B), I(T), I(H), I(Hkv),
                                         I(D), I(window), F(scale), I(is_bf16(qk))), "cpu_attn_fwd")
    return O, lse


def attn_bwd(qk, qkv, O, dO, lse, dqk, dqkv, B: int, T: int, H: int, Hkv: int, D: int, window: int):
    """Writes dQ|dK into ``dqk`` and dV into the value columns of ``dqkv``."""
    delta = torch.empty((B, H, T), dtype=torch.float32, device=qk.device)
    scale = 1.0 / math.sqrt(D)
    common = (P(qk), L(_ld(qk)), P(qkv), L(_ld(qkv)), P(O), L(_ld(O)), P(dO), L(_ld(dO)), P(lse), P(delta), P(dqk), L(_ld(dqk)),
              P(dqkv), L(_ld(dqkv)), I(B), I(T), I(H), I(Hkv), I(D), I(window), F(scale))
    if qk.is_cuda:
        lib = cuda_lib()
        if is_bf16(qk):
            check(lib.otb_attn_bwd(*common, P(_status(qk.device)), stream_ptr()), "attn_bwd")
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
    uniq, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
    seg = torch.zeros(uniq.numel() + 1, dtype=torch.int64, device=ids.device)
    torch.cumsum(counts, 0, out=seg[1:])
    order = order.contiguous()
    if dy.is_cuda:
        check(cuda_lib().otb_embedding_bwd(P(dy), P(order), P(seg), P(uniq), L(uniq.numel()), P(dW), I(dW.shape[1]), I(accumulate),
                                           I(is_bf16(dy)), stream_ptr()), "embedding_bwd")
    else:
        check(cpu_lib().otb_cpu_embedding_bwd(P(dy), P(order), P(seg), P(uniq), L(uniq.numel()), P(dW), I(dW.shape[1]), I(accumulate),
                                              I(is_bf16(dy))), "embedding_bwd")


# --------------------------------------------------------------------------- RoPE tables
_rope_cache: dict = {}


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [seq_len, head_dim/2] fp32. Always computed by the CPU routine (double precision,
    deterministic operations only) and copied, so every device holds the same bytes."""
    key = (seq_len, head_dim, float(theta))
    if key not in _rope_cache:
        half = head_dim // 2
        cos = torch.empty((seq_len, half), dtype=torch.float32)
        sin = torch.empty((seq_len, half), dtype=torch.float32)
        cpu_lib().otb_cpu_rope_tables(P(cos), P(sin), I(seq_len), I(half), _D(theta))
        _rope_cache[key] = (cos, sin)
    cos, sin = _rope_cache[key]
    return cos.to(device), sin.to(device)


def trunc_normal_(out: torch.Tensor, std: float, seed: int, offset: int) -> None:
    """Fill a CPU fp32 tensor from the Philox stream (element i <- stream word offset+i)."""
    assert out.device.type == "cpu" and out.dtype == torch.float32 and out.is_contiguous()
    cpu_lib().otb_cpu_trunc_normal(P(out), L(out.numel()), F(std), ctypes.c_uint64(seed), ctypes.c_uint64(offset))
