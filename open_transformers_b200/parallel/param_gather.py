"""Parameter all-gather fused into the consuming GEMM (``run.param_sharding: gather``).

With sharded ownership every process updates the rows of the weights it owns. In the default mode the AdamW kernel
stores the new bf16 rows into every GPU's weight buffer straight away - an NVLink-bound tail after the optimizer step.
In gather mode it stores them locally only, and the FIRST GEMM that multiplies by a weight after an update pulls the rows
of the other owners itself: four extra warps in each CTA of ``otb_pg_gemm`` copy runs of rows from the owners' buffers
(plain peer loads) into the local buffer and count them in, and the TMA producer of a tile waits for the counter of its own
B rows only - tiles over this process's rows start at once, the rest follow as their rows arrive. After that call the local
buffer holds the whole weight, so the other micro-batches and the backward pass run the plain GEMM on it.

This is what FSDP's parameter all-gather does before a layer's forward
(reference src/pretrain/parallel/parallelize_llama3_repop.py:198-202, Shard(0) row split src/pretrain/parallel/
deterministic_reduce.py:584-605), moved into the consumer. The bits are those of the plain GEMM: the copy moves bytes,
and every output element is still one ascending-k sum.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import native
from ..ops.native import I, L, P, check, cuda_lib, stream_ptr

EPI_BF16, EPI_F32, EPI_BF16_RES = 0, 1, 3


def flag_words(rows: int) -> int:
    """int32 words of counters a weight of ``rows`` rows needs (one per B tile of the GEMM plus one for the whole weight);
    zeroed once, they only grow."""
    tile = 256 if rows >= 256 else 128
    return -(-rows // tile) + 1


def uniform_rows_per_owner(row_ranges: list[tuple[int, int]], rows: int) -> int | None:
    """``row_ranges[p]`` = rows [lo, hi) of one weight held by process p (lo == hi: none). Returns r such that process p
    holds exactly rows [p*r, min((p+1)*r, rows)) - the only distribution the kernel's owner arithmetic covers, with the
    last process taking the remainder - or None."""
    if not row_ranges or row_ranges[0][0] != 0:
        return None
    r = row_ranges[0][1] - row_ranges[0][0]
    if r <= 0:
        return None
    n = len(row_ranges)
    for p, (lo, hi) in enumerate(row_ranges):
        want_lo = min(p * r, rows)
        want_hi = rows if p == n - 1 else min((p + 1) * r, rows)
        if hi <= lo:
            if want_hi > want_lo:
                return None
            continue
        if (lo, hi) != (want_lo, want_hi):
            return None
    return r


class GatheredWeight:
    """One weight, or up to three weights that are adjacent in the flat buffers (wq|wk|wv), as the B operand [N, K] of a
    forward GEMM whose rows are spread over the processes."""

    def __init__(self, local: torch.Tensor, peer_ptrs: list[int], rank: int, seg_begin: list[int], rows_per_owner: list[int],
                 flags: torch.Tensor):
        assert local.dim() == 2 and local.is_contiguous() and local.dtype == torch.bfloat16
        assert 1 <= len(seg_begin) == len(rows_per_owner) <= 3 and seg_begin[0] == 0
        assert flags.dtype == torch.int32 and flags.numel() >= flag_words(local.shape[0])
        self.local, self.rank, self.P = local, rank, len(peer_ptrs)
        self.flags = flags
        self._ptrs = (ctypes.c_void_p * self.P)(*peer_ptrs)
        self._seg = (ctypes.c_int * len(seg_begin))(*seg_begin)
        self._rpo = (ctypes.c_int * len(rows_per_owner))(*rows_per_owner)
        self._nseg = len(seg_begin)
        self.epoch_done = 0     # the update count whose rows are complete in the local buffer
        self.epoch = 0          # the update count of the owners' rows (set by the engine after each optimizer step)
        self.calls = 0

    def pending(self) -> bool:
        return self.epoch != self.epoch_done

    def mark_complete(self) -> None:
        self.epoch_done = self.epoch

    def gemm(self, x: torch.Tensor, residual: torch.Tensor | None = None, out_fp32: bool = False) -> torch.Tensor:
        """y[M, N] = x[M, K] W^T (+ residual), pulling the rows this process does not own on the way."""
        from ..ops.functional import _ld, _status

        M, K = x.shape
        N = self.local.shape[0]
        assert K == self.local.shape[1] and x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
        epi = EPI_F32 if out_fp32 else (EPI_BF16_RES if residual is not None else EPI_BF16)
        out = torch.empty((M, N), dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
        if residual is not None:
            assert residual.dtype == torch.bfloat16 and tuple(residual.shape) == (M, N)
        seq = self.calls + 1    # the counters of this weight have seen `calls` pulls so far
        check(cuda_lib().otb_pg_gemm(P(x), self._ptrs, P(self.flags), I(self.rank), I(self.P), ctypes.c_uint(seq), P(out), P(residual),
                                     I(M), I(N), I(K), L(_ld(x)), L(_ld(self.local)), L(_ld(out)), L(_ld(residual) if residual is not None else 0),
                                     self._seg, self._rpo, I(self._nseg), I(epi), P(_status(x.device)), stream_ptr()),
              "pg_gemm" if native._timing is None else "pg_gemm %dx%dx%d" % (M, N, K))
        self.mark_complete()
        self.calls += 1
        return out
