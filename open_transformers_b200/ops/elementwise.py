"""Tensor-level deterministic math for code outside the fused kernels (telemetry, schedules written with tensors,
experiments): ``exp``, ``log``, ``sqrt``, ``rsqrt``, ``sigmoid``, ``sin``, ``cos``, ``pow_int``, ``sum_dim``, ``mean_dim``,
``mean``. Every function evaluates the shared routines of ``csrc/common/det_math.h`` / ``det_reduce.h`` - fixed sequences of
correctly rounded IEEE operations - so a value has the same bits on every machine and device. They run on the CPU library;
a CUDA tensor is brought to the host, evaluated and copied back (CPU-authoritative, byte-copied, like the initialisation),
which is exact and adequate for the small tensors these helpers are for; the hot paths use the fused kernels instead.
(reference roles: repop.ops.exp / log / sqrt / pow / cos / sin / sum_dim / mean / mean_dim, used by
src/pretrain/model/z_loss.py:60-66, src/pretrain/model/modules/rope.py:31-94, src/pretrain/parallel/deterministic_reduce.py:581-817)"""
from __future__ import annotations

import torch

from .native import F, I, L, P, check, cpu_lib

_OPS = {"exp": 0, "log": 1, "sqrt": 2, "rsqrt": 3, "sigmoid": 4, "sin": 5, "cos": 6}


def _map(name: str, x: torch.Tensor) -> torch.Tensor:
    src = x.detach().to("cpu", torch.float32).contiguous()
    out = torch.empty_like(src)
    check(cpu_lib().otb_cpu_map(I(_OPS[name]), P(src), P(out), L(src.numel())), name)
    return out.to(device=x.device, dtype=x.dtype if x.dtype in (torch.float32, torch.bfloat16) else torch.float32)


def exp(x: torch.Tensor) -> torch.Tensor:
    return _map("exp", x)


def log(x: torch.Tensor) -> torch.Tensor:
    return _map("log", x)


def sqrt(x: torch.Tensor) -> torch.Tensor:
    return _map("sqrt", x)


def rsqrt(x: torch.Tensor) -> torch.Tensor:
    return _map("rsqrt", x)


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return _map("sigmoid", x)


def sin(x: torch.Tensor) -> torch.Tensor:
    return _map("sin", x)


def cos(x: torch.Tensor) -> torch.Tensor:
    return _map("cos", x)


def pow_int(x: torch.Tensor, n: int) -> torch.Tensor:
    """x ** n for a non-negative integer n by binary exponentiation: each step one correctly rounded multiply."""
    if n < 0 or int(n) != n:
        raise ValueError("pow_int takes a non-negative integer exponent")
    result, base, n = torch.ones_like(x), x.clone(), int(n)
    while n > 0:
        if n & 1:
            result = result * base
        base = base * base
        n >>= 1
    return result


def sum_dim(x: torch.Tensor, dim: int = -1, squares: bool = False, post_scale: float = 1.0) -> torch.Tensor:
    """Canonical fixed-order sum along ``dim`` (1024 interleaved partial sums combined by the block tree), fp32."""
    moved = x.detach().to("cpu", torch.float32).movedim(dim, -1).contiguous()
    rows, n = (moved.numel() // max(moved.shape[-1], 1), moved.shape[-1]) if moved.numel() else (0, 0)
    out = torch.zeros(moved.shape[:-1], dtype=torch.float32)
    if rows:
        check(cpu_lib().otb_cpu_row_sums(P(moved), L(rows), L(n), I(squares), F(post_scale), P(out)), "row_sums")
    return out.to(x.device)


def mean_dim(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Mean along ``dim``: the canonical sum times the host reciprocal 1/n (never a division by a Python scalar)."""
    return sum_dim(x, dim, post_scale=1.0 / x.shape[dim])


def mean(x: torch.Tensor) -> torch.Tensor:
    return sum_dim(x.reshape(-1), 0, post_scale=1.0 / max(x.numel(), 1))
