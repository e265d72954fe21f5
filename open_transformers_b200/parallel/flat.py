"""Flat parameter layout, virtual-shard segments and the chunk table shared by the fused
reduce / AdamW kernels and their CPU twins; plus peer-mapped flat buffers (CUDA IPC).

Layout rules
* parameters are laid out in ``named_parameters()`` order, each starting at a multiple of 64
  elements (wq|wk|wv stay back to back, so one GEMM reads them as a single [3072, 2048] weight);
* virtual shard ``s`` of a parameter is its logical ``Shard(0)`` row range (ceil split, the layout
  FSDP2 uses: reference src/pretrain/parallel/deterministic_reduce.py:584-621);
* a *segment* is (parameter, shard); segments are ordered shard-major and cut into chunks of at
  most 8192 elements that never straddle a segment; GPUs own contiguous runs of whole segments.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import numpy as np
import torch

CHUNK = 8192
ALIGN = 64


def shard_rows(dim0: int, num_shards: int, shard: int) -> tuple[int, int]:
    fcs = -(-dim0 // num_shards)
    lo = min(shard * fcs, dim0)
    return lo, min((shard + 1) * fcs, dim0)


@dataclass
class Segment:
    param: int
    shard: int
    start: int      # flat element offset
    length: int
    first_chunk: int = 0
    n_chunks: int = 0


@dataclass
class FlatLayout:
    names: list[str]
    shapes: list[tuple[int, ...]]
    offsets: list[int]
    numels: list[int]
    total: int
    num_shards: int
    groups: list[int]                      # 0 = weight decay, 1 = no decay, per parameter
    segments: list[Segment] = field(default_factory=list)
    chunk_start: np.ndarray | None = None  # int64 [C]
    chunk_len: np.ndarray | None = None    # int32 [C]
    chunk_group: np.ndarray | None = None  # int32 [C]
    seg_first: np.ndarray | None = None    # int32 [S+1]

    @classmethod
    def build(cls, named_shapes: list[tuple[str, tuple[int, ...]]], num_shards: int, groups: list[int]) -> "FlatLayout":
        names, shapes, offsets, numels = [], [], [], []
        off = 0
        for name, shape in named_shapes:
            n = int(np.prod(shape)) if len(shape) else 1
            names.append(name); shapes.append(tuple(shape)); offsets.append(off); numels.append(n)
            off += -(-n // ALIGN) * ALIGN
        lay = cls(names, shapes, offsets, numels, off, num_shards, list(groups))
        cs, cl, cg, sf = [], [], [], [0]
        for s in range(num_shards):
            for pi, shape in enumerate(shapes):
                dim0 = shape[0] if len(shape) else 1
                row = numels[pi] // max(dim0, 1)
                lo, hi = shard_rows(dim0, num_shards, s)
                if hi <= lo:
                    continue
                seg = Segment(pi, s, offsets[pi] + lo * row, (hi - lo) * row, first_chunk=len(cs))
                for c0 in range(0, seg.length, CHUNK):
                    cs.append(seg.start + c0); cl.append(min(CHUNK, seg.length - c0)); cg.append(groups[pi])
                seg.n_chunks = len(cs) - seg.first_chunk
                sf.append(len(cs))
                lay.segments.append(seg)
        lay.chunk_start = np.asarray(cs, dtype=np.int64)
        lay.chunk_len = np.asarray(cl, dtype=np.int32)
        lay.chunk_group = np.asarray(cg, dtype=np.int32)
        lay.seg_first = np.asarray(sf, dtype=np.int32)
        for seg in lay.segments:
            if seg.start % 4:
                raise ValueError("segment of %s shard %d starts at unaligned element %d (row size must be a multiple of 4)"
                                 % (names[seg.param], seg.shard, seg.start))
        return lay

    def owner_ranges(self, world: int) -> list[tuple[int, int]]:
        """Contiguous runs of whole segments per physical rank, balanced by element count: [(seg_lo, seg_hi)]."""
        total = sum(s.length for s in self.segments)
        owner, cum = [], 0
        for seg in self.segments:
            owner.append(min(world - 1, int((cum + seg.length / 2) * world / total)))
            cum += seg.length
        out = []
        for r in range(world):
            idx = [i for i, o in enumerate(owner) if o == r]
            out.append((idx[0], idx[-1] + 1) if idx else (0, 0))
        return out

    def view(self, flat: torch.Tensor, i: int) -> torch.Tensor:
        return flat[self.offsets[i]: self.offsets[i] + self.numels[i]].view(self.shapes[i])


class _CudaPtr:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap memory this process mapped."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def lazy_zeros(n: int, dtype: torch.dtype, device) -> torch.Tensor:
    """``torch.zeros`` for the large flat buffers. On the CPU the tensor sits on an anonymous memory mapping: pages exist
    only once they are read or written, so a buffer that is never used (the gradient buffers of an init audit, which runs no
    step) costs neither time nor resident memory, where ``torch.zeros`` writes every byte up front. The tensor keeps the
    mapping alive. Device tensors, and small ones, are plain ``torch.zeros``."""
    device = torch.device(device)
    nbytes = n * dtype.itemsize
    if device.type != "cpu" or nbytes < (1 << 24):
        return torch.zeros(n, dtype=dtype, device=device)
    import mmap

    try:
        return torch.frombuffer(mmap.mmap(-1, nbytes), dtype=dtype, count=n)
    except (OSError, ValueError):   # no anonymous mapping of that size on this system: the ordinary allocation reports the error
        return torch.zeros(n, dtype=dtype, device=device)


class PeerBuffer:
    """A flat device buffer every rank of ``group`` can address: ``ptrs[r]`` is rank r's buffer as
    seen from this process (CUDA IPC mapping for r != rank). On the CPU, or with a single rank, it is
    an ordinary tensor."""

    def __init__(self, nbytes: int, device: torch.device, rank: int = 0, world: int = 1, group=None, storage: torch.Tensor | None = None):
        self.nbytes, self.device, self.rank, self.world = nbytes, device, rank, world
        self._peer_ptrs: list[int] = []
        self._own_ptr = 0
        self._group = group
        self._ipc = device.type == "cuda" and world > 1
        if storage is not None:  # caller-provided bytes (a file mapping): single rank only
            assert not self._ipc and storage.dtype == torch.uint8 and storage.numel() >= nbytes
        if not self._ipc:
            self.bytes = storage[:nbytes] if storage is not None else lazy_zeros(nbytes, torch.uint8, device)
            self.ptrs = [self.bytes.data_ptr()]
            return
        import torch.distributed as dist

        from ..ops.native import check, cuda_lib

        lib = cuda_lib()
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.otb_ipc_alloc(ctypes.c_size_t(nbytes), ctypes.byref(ptr), handle), "ipc_alloc")
        self._own_ptr = ptr.value
        self.bytes = torch.as_tensor(_CudaPtr(ptr.value, nbytes), device=device)
        handles: list = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(ptr.value)
                continue
            h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
            pp = ctypes.c_void_p()
            check(lib.otb_ipc_open(h, ctypes.byref(pp)), "ipc_open (rank %d)" % r)
            self.ptrs.append(pp.value)
            self._peer_ptrs.append(pp.value)

    def typed(self, dtype: torch.dtype) -> torch.Tensor:
        return self.bytes.view(dtype)

    def close(self) -> None:
        if self._ipc:
            from ..ops.native import cuda_lib

            import torch.distributed as dist

            lib = cuda_lib()
            torch.cuda.synchronize()
            for p in self._peer_ptrs:
                lib.otb_ipc_close(ctypes.c_void_p(p))
            self._peer_ptrs = []
            if self._own_ptr:
                # every rank unmaps its view of the others' buffers before any owner frees its memory
                if dist.is_initialized():
                    dist.barrier(group=self._group)
                self.bytes = None
                lib.otb_ipc_free(ctypes.c_void_p(self._own_ptr))
                self._own_ptr = 0
