"""Tensor parallelism with sequence-parallel activations over NVLink peer memory.

A tensor-parallel group of P ranks (one process per GPU) splits every block's weights the Megatron way and keeps
the residual stream sharded by tokens. The two communication patterns are each ONE hand-written kernel
(``csrc/cuda/gemm_tc05.cu``), never a library collective:

* ``ag_gemm``  - all-gather -> GEMM (column-parallel layers: QKV, gate/up; and the data-gradient of row-parallel
  layers). A few CTAs of the launch push this rank's token rows into every peer's full-size activation buffer with
  plain peer stores and raise a flag per 128-row block; the tensor-core CTAs start on the local rows and wait, block
  by block, for the peers' rows.
* ``chain_gemm`` - GEMM -> ordered reduction (row-parallel layers: attention output, down projection; and the
  data-gradient of column-parallel layers). The K-split partial sums are not added afterwards: the fp32
  accumulator tile travels rank 0 -> 1 -> ... -> P-1 and every rank continues the same ascending-k tensor-core
  accumulation in tensor memory, so the result has exactly the bits of the unsplit single-GPU GEMM; the last rank
  stores each tile into the memory of the rank that owns those token rows, where ``finish`` applies the residual add.

Because neither pattern changes a single rounding, a tensor-parallel run hashes like the data-parallel run of the
same virtual topology and like the single-device replay.

All buffers that a peer reads or writes are CUDA-IPC allocations created once (``TpWorkspace``); flags are
epoch-numbered so nothing is ever reset, and every wait inside a kernel is bounded and reports through the status
word (``ops.functional.kernel_status``). (The reference removed its tensor-parallel path, README.md:231-234; this
module has no counterpart there.)
"""
from __future__ import annotations

import ctypes

import torch

from ..ops.functional import _status
from ..ops.native import I, L, P as PTR, check, cuda_lib, stream_ptr
from .flat import PeerBuffer

BM = 128  # row-block of the GEMM kernels and of the all-gather flags


def _ptrs(values):
    arr = (ctypes.c_void_p * len(values))()
    for i, v in enumerate(values):
        arr[i] = v
    return arr


class _Site:
    """One gathered-activation buffer [M, K] (bf16) with its flags and call counter."""

    def __init__(self, ws: "TpWorkspace", M: int, K: int):
        self.M, self.K = M, K
        self.buf = PeerBuffer(M * K * 2, ws.device, ws.rank, ws.P, ws.group)
        self.flags = PeerBuffer(4 * ws.P * (M // BM // ws.P), ws.device, ws.rank, ws.P, ws.group)
        self.full = self.buf.typed(torch.bfloat16).view(M, K)
        self.seq = 0


class _Chain:
    """Inbox and result buffers [M, N] fp32 of the chained GEMM with their flags and call counter."""

    def __init__(self, ws: "TpWorkspace", M: int, N: int):
        bn = cuda_lib().otb_tp_chain_bn(I(N))
        tiles = (M // BM) * ((N + bn - 1) // bn)
        self.M, self.N = M, N
        self.inbox = PeerBuffer(M * N * 4, ws.device, ws.rank, ws.P, ws.group)
        self.result = PeerBuffer(M * N * 4, ws.device, ws.rank, ws.P, ws.group)
        self.inbox_flags = PeerBuffer(16 * tiles, ws.device, ws.rank, ws.P, ws.group)
        self.result_flags = PeerBuffer(16 * tiles, ws.device, ws.rank, ws.P, ws.group)
        self.seq = 0


class TpWorkspace:
    """Peer-visible buffers of one tensor-parallel group. ``rank``/``P`` are the position in and size of the group
    (``group`` is the matching torch.distributed group, used only to exchange IPC handles)."""

    def __init__(self, device, rank: int, P: int, group=None, copier_ctas: int = 16):
        self.device, self.rank, self.P, self.group = torch.device(device), rank, P, group
        self.copier_ctas = copier_ctas
        self.lib = cuda_lib()
        self._sites: dict = {}
        self._chains: dict = {}
        self._bar = PeerBuffer(4 * 8, self.device, rank, P, group)
        self._bar_seq = 0

    # ------------------------------------------------------------------ buffers
    def site(self, key, M: int, K: int) -> _Site:
        s = self._sites.get(key)
        if s is None or (s.M, s.K) != (M, K):
            assert M % (self.P * BM) == 0, "token count must be a multiple of %d" % (self.P * BM)
            s = self._sites[key] = _Site(self, M, K)
        return s

    def chain(self, key, M: int, N: int) -> _Chain:
        c = self._chains.get(key)
        if c is None or (c.M, c.N) != (M, N):
            assert M % (self.P * BM) == 0
            c = self._chains[key] = _Chain(self, M, N)
        return c

    def shard_rows(self, M: int) -> slice:
        per = M // self.P
        return slice(self.rank * per, (self.rank + 1) * per)

    # --------------------------------------------------------------- collectives
    def barrier(self) -> None:
        """Cross-GPU barrier on the current stream (flag exchange over peer memory, bounded wait)."""
        self._bar_seq += 1
        check(self.lib.otb_peer_barrier(_ptrs(self._bar.ptrs), I(self.rank), I(self.P), ctypes.c_uint(self._bar_seq),
                                        PTR(_status(self.device)), stream_ptr()), "peer_barrier")

    def ag_gemm(self, key, x_shard: torch.Tensor, w: torch.Tensor, b_mn: bool = False, out_dtype=torch.bfloat16):
        """``C[M, N] = all_gather(x_shard)[M, K] @ op(w)^T``; returns ``(C, x_full)`` where ``x_full`` is the gathered
        activation (kept for the weight-gradient GEMM). ``w``: [N, K], or [K, N] with ``b_mn``."""
        rows, K = x_shard.shape
        M = rows * self.P
        N = w.shape[1] if b_mn else w.shape[0]
        s = self.site(key, M, K)
        mine = s.full[self.shard_rows(M)]
        if x_shard.data_ptr() != mine.data_ptr():  # a producer may write its rows straight into ``site(...).full``
            mine.copy_(x_shard)
        s.seq += 1
        C = torch.empty((M, N), dtype=out_dtype, device=self.device)
        epi = 0 if out_dtype == torch.bfloat16 else 1
        check(self.lib.otb_tp_ag_gemm(_ptrs(s.buf.ptrs), _ptrs(s.flags.ptrs), I(self.rank), I(self.P), ctypes.c_uint(s.seq), PTR(w), PTR(C),
                                      I(M), I(N), I(K), L(w.stride(0)), L(C.stride(0)), I(b_mn), I(epi), I(self.copier_ctas),
                                      PTR(_status(self.device)), stream_ptr()), "tp_ag_gemm")
        return C, s.full

    def chain_gemm(self, key, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False, residual_shard: torch.Tensor | None = None):
        """This rank's K slice of ``y = A W^T (+ residual)``: ``a`` [M, K/P], ``w`` [N, K/P] (or [K/P, N] with
        ``b_mn``). Returns this rank's token rows of y, [M/P, N] bf16, bit-identical to the unsplit GEMM."""
        M, Kr = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        c = self.chain(key, M, N)
        c.seq += 1
        last = self.rank == self.P - 1
        if last:
            outs, oflags = c.result.ptrs, c.result_flags.ptrs
        else:
            outs, oflags = [c.inbox.ptrs[self.rank + 1]], [c.inbox_flags.ptrs[self.rank + 1]]
        st = PTR(_status(self.device))
        check(self.lib.otb_tp_chain_gemm(PTR(a), PTR(w), I(M), I(N), I(Kr), L(a.stride(0)), L(w.stride(0)), I(b_mn),
                                         ctypes.c_void_p(c.inbox.ptrs[self.rank]), ctypes.c_void_p(c.inbox_flags.ptrs[self.rank]),
                                         _ptrs(outs), _ptrs(oflags), L(N), I(self.rank), I(self.P), ctypes.c_uint(c.seq), st, stream_ptr()),
              "tp_chain_gemm")
        y = torch.empty((M // self.P, N), dtype=torch.bfloat16, device=self.device)
        check(self.lib.otb_tp_finish(ctypes.c_void_p(c.result.ptrs[self.rank]), ctypes.c_void_p(c.result_flags.ptrs[self.rank]),
                                     ctypes.c_uint(c.seq), PTR(residual_shard), PTR(y), I(M), I(N), I(self.rank), I(self.P), L(N),
                                     L(residual_shard.stride(0) if residual_shard is not None else 0), L(y.stride(0)), st, stream_ptr()),
              "tp_finish")
        return y

    def close(self) -> None:
        for s in self._sites.values():
            s.full = None
            s.buf.close()
            s.flags.close()
        for c in self._chains.values():
            for b in (c.inbox, c.result, c.inbox_flags, c.result_flags):
                b.close()
        self._bar.close()
        self._sites, self._chains = {}, {}
