"""Chained blake2b-256 state hash: byte layout, sharded combine, running batch digest.

Wire formats (NUL-delimited fields; dtype strings are torch's ``str(dtype)``, shapes Python's
``str(tuple)``), equal to the reference's (src/pretrain/train/state_hash.py:233-528):

v2 "full" (init hash, ``hash_ckpt``)::

    b"pretrain.state_hash.v2\\n" b"prev\\0" prev32 b"params\\0"
    for name, p in sorted(named_parameters):
        name b"\\0" TENSOR("weight", p)
        [b"optim_step\\0" int64-LE  TENSOR("optim_exp_avg") TENSOR("optim_exp_avg_sq") [TENSOR("optim_max_exp_avg_sq")]]
        [b"grad_none\\0" | TENSOR("grad", grad)]
    [b"param_groups\\0" json] [b"batch_digest\\0" digest32]

v3 "sharded" (every periodic / checkpoint hash): one digest per virtual shard over that shard's
logical ``Shard(0)`` rows of every parameter (same per-parameter record, shard shape), combined
rank-major ``blake2b(local[r % num_shards] for r in range(num_ranks))`` and finalised as::

    b"pretrain.state_hash.v3\\n" b"prev\\0" prev32 b"shard_state\\0" d32 b"param_groups\\0" json b"batch_digest\\0" d32

TENSOR(tag, t) = tag b"\\0" dtype b"\\0" shape b"\\0" raw-bytes. With ``tensor_digest="tree"`` the
raw bytes are replaced by b"tree\\0" + the 32-byte blake2b tree digest of those bytes (4096-byte
leaves, csrc/common/blake2b.h), which a GPU computes in parallel; the rest of the layout is
unchanged.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
from typing import Any, Iterable, Mapping, Sequence

import numpy as np
import torch

DIGEST_SIZE = 32
V2_TAG = b"pretrain.state_hash.v2\n"
V3_TAG = b"pretrain.state_hash.v3\n"
ZERO_DIGEST = b"\0" * DIGEST_SIZE
MOMENT_KEYS = ("exp_avg", "exp_avg_sq", "max_exp_avg_sq")


def _new():
    return hashlib.blake2b(digest_size=DIGEST_SIZE)


def tensor_bytes(t: torch.Tensor) -> bytes:
    """Raw little-endian bytes of a tensor (any dtype, bf16 included), via a CPU contiguous copy."""
    t = t.detach().to("cpu").contiguous()
    if t.numel() == 0:
        return b""
    return t.view(torch.uint8).numpy().tobytes() if t.dim() > 0 else t.reshape(1).view(torch.uint8).numpy().tobytes()


FEED_CHUNK = 1 << 26


def feed_raw(h, t: torch.Tensor) -> None:
    """``h.update`` over a tensor's raw little-endian bytes without building a ``bytes`` copy of it: the hash reads the
    tensor's own memory (a host copy first, for a device tensor) in 64 MB pieces. The digest is that of
    ``h.update(tensor_bytes(t))``; for the 19 GB of weights and moments of a 1.6 B-parameter model the copy was most of the time
    and all of the extra memory of a full hash."""
    t = t.detach().to("cpu").contiguous()
    if t.numel() == 0:
        return
    flat = t.reshape(-1).view(torch.uint8).numpy()
    for at in range(0, flat.size, FEED_CHUNK):
        h.update(flat[at:at + FEED_CHUNK])


def tree_digest_bytes(data: bytes | np.ndarray) -> bytes:
    """32-byte tree digest of a byte string (host implementation)."""
    from ..ops.native import cpu_lib

    arr = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1).view(np.uint8)
    if not (arr.flags["C_CONTIGUOUS"] and arr.ctypes.data % 8 == 0 and arr.size > 0):
        buf = np.empty(arr.size + 8, dtype=np.uint8)  # the native routine wants 8-byte aligned input; numpy allocations are 16-byte aligned
        buf[: arr.size] = arr
        src = buf
    else:
        src = arr  # tensors and aligned arrays are digested in place: no copy of the state
    out = (ctypes.c_ubyte * 32)()
    cpu_lib().otb_cpu_tree_digest(src.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(arr.size), out)
    return bytes(out)


def tree_digest_tensor(t: torch.Tensor, scratch: dict | None = None) -> bytes:
    """Tree digest of a tensor's bytes; runs on the GPU for CUDA tensors."""
    t = t.detach().contiguous()
    if not t.is_cuda:
        return tree_digest_bytes(t.reshape(-1).view(torch.uint8).numpy())
    from ..ops.native import P, check, cuda_lib, stream_ptr

    lib = cuda_lib()
    nbytes = t.numel() * t.element_size()
    lib.otb_tree_digest_scratch.restype = ctypes.c_uint64
    need = int(lib.otb_tree_digest_scratch(ctypes.c_uint64(nbytes)))
    sc = torch.empty(need, dtype=torch.uint8, device=t.device)
    out = torch.empty(32, dtype=torch.uint8, device=t.device)
    check(lib.otb_tree_digest(P(t), ctypes.c_uint64(nbytes), P(sc), ctypes.c_uint64(need), P(out), stream_ptr()), "tree_digest")
    return bytes(out.cpu().numpy().tobytes())


_batch_work: dict = {}


def tree_digest_batch(tensors) -> list[bytes]:
    """Tree digests of many tensors; CUDA tensors of one device go through a single batched launch per
    tree level and one device-to-host copy of all digests."""
    tensors = [t.detach() for t in tensors]
    if not tensors:
        return []
    if not tensors[0].is_cuda:
        return [tree_digest_tensor(t) for t in tensors]
    from ..ops.native import P, check, cuda_lib, stream_ptr

    lib = cuda_lib()
    n = len(tensors)
    for t in tensors:
        assert t.is_contiguous() and t.is_cuda
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
    lens = (ctypes.c_uint64 * n)(*[t.numel() * t.element_size() for t in tensors])
    lib.otb_tree_digest_batch_work.restype = ctypes.c_uint64
    need = int(lib.otb_tree_digest_batch_work(lens, ctypes.c_int(n)))
    dev = tensors[0].device
    work = _batch_work.get(dev)
    if work is None or work.numel() < need:
        work = torch.empty(need, dtype=torch.uint8, device=dev)
        _batch_work[dev] = work
    out = torch.empty(n * 32, dtype=torch.uint8, device=dev)
    check(lib.otb_tree_digest_batch(ptrs, lens, ctypes.c_int(n), P(work), ctypes.c_uint64(work.numel()), P(out), stream_ptr()),
          "tree_digest_batch")
    raw = out.cpu().numpy().tobytes()
    return [raw[i * 32:(i + 1) * 32] for i in range(n)]


class TreeDigestPlan:
    """Tree digests of a FIXED set of CUDA tensors (same addresses and sizes every time, like the flat state buffers
    of a training run), launched without any host synchronisation so they can run on a side stream under the next
    step's compute. ``launch(stream)`` enqueues the level kernels and the copy of the n x 32 digest bytes into pinned
    host memory; ``digests()`` (after the caller has waited for the stream or an event) returns them."""

    MAX_LEVELS = 8

    def __init__(self, tensors):
        from ..ops.native import P, cuda_lib

        tensors = [t.detach() for t in tensors]
        assert tensors and all(t.is_cuda and t.is_contiguous() for t in tensors)
        self._keep = tensors
        lib = cuda_lib()
        n = self.n = len(tensors)
        dev = tensors[0].device
        ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
        lens = (ctypes.c_uint64 * n)(*[t.numel() * t.element_size() for t in tensors])
        lib.otb_tree_digest_scratch.restype = ctypes.c_uint64
        need = sum(int(lib.otb_tree_digest_scratch(ctypes.c_uint64(l))) for l in lens)
        self.work = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        lib.otb_tree_plan_words.restype = ctypes.c_uint64
        words = int(lib.otb_tree_plan_words(ctypes.c_int(n)))
        tab = np.zeros(words, dtype=np.uint64)
        self.level_leaves = (ctypes.c_uint64 * self.MAX_LEVELS)()
        lib.otb_tree_plan.restype = ctypes.c_long
        levels = int(lib.otb_tree_plan(ptrs, lens, ctypes.c_int(n), P(self.work), ctypes.c_uint64(self.work.numel()),
                                       tab.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(words), self.level_leaves,
                                       ctypes.c_int(self.MAX_LEVELS)))
        if levels < 0:
            raise RuntimeError("tree digest plan failed with code %d" % levels)
        self.levels = levels
        self.tab = torch.from_numpy(tab.view(np.int64)).to(dev)
        self.out = torch.empty(n * 32, dtype=torch.uint8, device=dev)
        self.host = torch.empty(n * 32, dtype=torch.uint8).pin_memory()

    def launch(self, stream=None) -> None:
        from ..ops.native import P, check, cuda_lib

        st = stream if stream is not None else torch.cuda.current_stream()
        with torch.cuda.stream(st):
            check(cuda_lib().otb_tree_run(P(self.tab), ctypes.c_int(self.n), ctypes.c_int(self.levels), self.level_leaves, P(self.out),
                                          ctypes.c_void_p(st.cuda_stream)), "tree_digest_plan")
            self.host.copy_(self.out, non_blocking=True)

    def digests(self) -> list[bytes]:
        raw = self.host.numpy().tobytes()
        return [raw[i * 32:(i + 1) * 32] for i in range(self.n)]


def _prev_bytes(prev: bytes | str | None) -> bytes:
    if prev is None:
        return ZERO_DIGEST
    if isinstance(prev, str):
        prev = bytes.fromhex(prev)
    prev = bytes(prev)
    # a shorter digest is zero-padded, a longer one truncated (reference src/pretrain/train/state_hash.py:116-127)
    return prev + b"\0" * (DIGEST_SIZE - len(prev)) if len(prev) < DIGEST_SIZE else prev[:DIGEST_SIZE]


def feed_tensor(h, tag: str, t: torch.Tensor, tensor_digest: str = "raw", precomputed: bytes | None = None) -> None:
    h.update(tag.encode() + b"\0")
    h.update(str(t.dtype).encode() + b"\0")
    h.update(str(tuple(t.shape)).encode() + b"\0")
    if tensor_digest == "tree":
        h.update(b"tree\0")
        h.update(precomputed if precomputed is not None else tree_digest_tensor(t))
    else:
        feed_raw(h, t)


def param_groups_json(param_groups: Sequence[Mapping[str, Any]]) -> bytes:
    slim = [{k: v for k, v in g.items() if k != "params"} for g in param_groups]
    return json.dumps(slim, sort_keys=True, default=str).encode()


def feed_param_record(h, name: str, weight: torch.Tensor, state: Mapping[str, Any] | None, grad, include_grads: bool,
                      tensor_digest: str = "raw") -> None:
    """One parameter's record: name, weight, optimizer step + moments (if any), gradient."""
    h.update(name.encode() + b"\0")
    feed_tensor(h, "weight", weight, tensor_digest)
    if state:
        step = state.get("step", 0)
        step = int(step.item()) if isinstance(step, torch.Tensor) else int(step)
        h.update(b"optim_step\0" + int(step).to_bytes(8, "little", signed=True))
        for key in MOMENT_KEYS:
            v = state.get(key)
            if isinstance(v, torch.Tensor):
                feed_tensor(h, "optim_" + key, v, tensor_digest)
    if include_grads:
        if grad is None:
            h.update(b"grad_none\0")
        else:
            feed_tensor(h, "grad", grad, tensor_digest)


def compute_state_hash(named_params: Iterable[tuple[str, torch.Tensor]], optimizer_state: Mapping[str, Mapping] | None = None,
                       param_groups: Sequence[Mapping] | None = None, *, prev: bytes | str | None = None,
                       include_grads: bool = False, grads: Mapping[str, torch.Tensor | None] | None = None,
                       batch_digest: bytes | None = None, tensor_digest: str = "raw") -> str:
    """v2 full-tensor hash (hex)."""
    h = _new()
    h.update(V2_TAG)
    h.update(b"prev\0" + _prev_bytes(prev))
    h.update(b"params\0")
    for name, p in sorted(named_params, key=lambda kv: kv[0]):
        st = optimizer_state.get(name) if optimizer_state else None
        g = None
        if include_grads:
            g = grads.get(name) if grads is not None else getattr(p, "grad", None)
        feed_param_record(h, name, p.detach() if isinstance(p, torch.Tensor) else p, st, g, include_grads, tensor_digest)
    if param_groups is not None:
        h.update(b"param_groups\0" + param_groups_json(param_groups))
    if batch_digest is not None:
        h.update(b"batch_digest\0" + batch_digest)
    return h.hexdigest()


def shard_rows(dim0: int, num_shards: int, shard: int) -> tuple[int, int]:
    """Logical (unpadded) ``Shard(0)`` row range of ``shard``: ceil split, empty tail shards allowed."""
    fcs = -(-dim0 // num_shards)
    lo = min(shard * fcs, dim0)
    return lo, min((shard + 1) * fcs, dim0)


def shard_view(t: torch.Tensor, num_shards: int, shard: int) -> torch.Tensor:
    if t.dim() == 0:
        t = t.reshape(1)
    lo, hi = shard_rows(t.shape[0], num_shards, shard)
    return t[lo:hi]


def local_shard_state_digest(named_params: Iterable[tuple[str, torch.Tensor]], optimizer_state, grads, num_shards: int,
                             shard: int, include_grads: bool = True, tensor_digest: str = "raw") -> bytes:
    """Digest of virtual shard ``shard``: per-parameter records over that shard's rows."""
    h = _new()
    for name, p in sorted(named_params, key=lambda kv: kv[0]):
        st = optimizer_state.get(name) if optimizer_state else None
        sst = None
        if st:
            sst = {"step": st.get("step", 0)}
            for key in MOMENT_KEYS:
                if isinstance(st.get(key), torch.Tensor):
                    sst[key] = shard_view(st[key], num_shards, shard)
        g = grads.get(name) if grads is not None else None
        gs = shard_view(g, num_shards, shard) if g is not None else None
        feed_param_record(h, name, shard_view(p.detach(), num_shards, shard), sst, gs, include_grads, tensor_digest)
    return h.digest()


def combine_shard_state(local_digests: Sequence[bytes], num_ranks: int) -> bytes:
    """Rank-major wrap: rank r contributes the digest of shard r % num_shards."""
    n = len(local_digests)
    h = _new()
    for r in range(num_ranks):
        h.update(local_digests[r % n])
    return h.digest()


def finalize_state_hash(shard_state: bytes, param_groups: Sequence[Mapping] | None, prev: bytes | str | None,
                        batch_digest: bytes | None) -> str:
    """v3 stream: tag, prev, shard_state, then `param_groups` only when there is an optimizer and `batch_digest` only
    when one is given (reference src/pretrain/train/state_hash.py:492-528)."""
    if len(shard_state) != DIGEST_SIZE:
        raise ValueError("shard_state must be %d bytes, got %d" % (DIGEST_SIZE, len(shard_state)))
    h = _new()
    h.update(V3_TAG)
    h.update(b"prev\0" + _prev_bytes(prev))
    h.update(b"shard_state\0" + shard_state)
    if param_groups is not None:
        h.update(b"param_groups\0" + param_groups_json(param_groups))
    if batch_digest is not None:
        if len(batch_digest) != DIGEST_SIZE:
            raise ValueError("batch_digest must be %d bytes, got %d" % (DIGEST_SIZE, len(batch_digest)))
        h.update(b"batch_digest\0" + batch_digest)
    return h.hexdigest()


def audit_shard_state_digest(named_params, optimizer_state, grads, num_shards: int, num_ranks: int,
                             include_grads: bool = True, tensor_digest: str = "raw") -> bytes:
    """Single-process reconstruction of the cluster's shard_state from full tensors."""
    named = list(named_params)
    locals_ = [local_shard_state_digest(named, optimizer_state, grads, num_shards, s, include_grads, tensor_digest)
               for s in range(num_shards)]
    return combine_shard_state(locals_, num_ranks)


class RunningBatchHasher:
    """Per-rank chain over every batch consumed: chain_n = blake2b(chain_{n-1} || records of the batch's
    tensors sorted by key). The chain value is the whole state, so it can be checkpointed as 32 bytes."""

    def __init__(self, prev_digest: bytes | None = None):
        if prev_digest is not None and len(prev_digest) != DIGEST_SIZE:
            raise ValueError("prev_digest must be %d bytes" % DIGEST_SIZE)
        self._chain = bytes(prev_digest) if prev_digest is not None else ZERO_DIGEST

    def update(self, batch: Mapping[str, torch.Tensor]) -> None:
        h = _new()
        h.update(self._chain)
        for k in sorted(batch):
            t = batch[k]
            h.update(k.encode() + b"\0" + str(t.dtype).encode() + b"\0" + str(tuple(t.shape)).encode() + b"\0")
            feed_raw(h, t)
        self._chain = h.digest()

    def local_digest(self) -> bytes:
        return self._chain


def combine_batch_digests(digests: Sequence[bytes]) -> bytes:
    if not digests:
        raise ValueError("no batch digests")
    if any(len(d) != DIGEST_SIZE for d in digests):
        raise ValueError("batch digests must be %d bytes" % DIGEST_SIZE)
    if len(digests) == 1:
        return bytes(digests[0])
    h = _new()
    for d in digests:
        h.update(d)
    return h.digest()


def all_gather_bytes(payload: bytes, group=None) -> list[bytes]:
    """Gather equal-length byte strings from every rank of ``group`` (a gloo/NCCL group) in rank order."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return [payload]
    objs: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(objs, payload, group=group)
    return objs
