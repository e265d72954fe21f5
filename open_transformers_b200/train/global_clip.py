"""Stateless global-norm gradient clipping.

    h = min( max_norm / (||g|| + 1e-6), 1 )        all in fp32, tensor / tensor, never tensor / python scalar
    g <- g * h                                     per local shard

``||g||`` is the deterministic norm: squared-norm partials per (parameter, virtual shard) in the
canonical chunk order, summed ascending shard then ascending parameter, then sqrt
(``grad_norm_algo = deterministic_per_tensor_sos_v1``). The training engine applies ``h`` inside the
fused AdamW kernel; these helpers serve the replay, tests and plain-tensor users
(reference src/pretrain/train/global_clip.py:47-79).
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops.native import I, P, check, cpu_lib, cuda_lib, stream_ptr
from ..parallel.flat import FlatLayout

EPS = 1e-6


def clip_coefficient(total_norm: float, max_norm: float) -> float:
    if max_norm <= 0:
        return 1.0
    h = np.float32(max_norm) / np.float32(np.float32(total_norm) + np.float32(EPS))
    return float(min(h, np.float32(1.0)))


def deterministic_global_norm(named_grads: list[tuple[str, torch.Tensor]], num_shards: int) -> tuple[float, np.ndarray]:
    """Norm of a list of full gradients (same device, fp32) with the cluster's association."""
    named_grads = [(n, g) for n, g in named_grads if g is not None]
    lay = FlatLayout.build([(n, tuple(g.shape)) for n, g in named_grads], num_shards, [0] * len(named_grads))
    dev = named_grads[0][1].device
    flat = torch.zeros(lay.total, dtype=torch.float32, device=dev)
    for i, (_, g) in enumerate(named_grads):
        lay.view(flat, i).copy_(g.detach().to(torch.float32))
    cs, cl, sf = (torch.from_numpy(a).to(dev) for a in (lay.chunk_start, lay.chunk_len, lay.seg_first))
    sos = torch.zeros(len(lay.chunk_start), dtype=torch.float32, device=dev)
    seg = torch.zeros(len(lay.segments), dtype=torch.float32, device=dev)
    if dev.type == "cuda":
        lib = cuda_lib()
        check(lib.otb_chunk_sos(P(flat), P(cs), P(cl), I(len(lay.chunk_start)), P(sos), stream_ptr()), "chunk_sos")
        check(lib.otb_seg_pair_tree(P(sos), P(sf), I(len(lay.segments)), P(seg), stream_ptr()), "seg_tree")
    else:
        lib = cpu_lib()
        check(lib.otb_cpu_chunk_sos(P(flat), P(cs), P(cl), I(len(lay.chunk_start)), P(sos)), "chunk_sos")
        check(lib.otb_cpu_seg_pair_tree(P(sos), P(sf), I(len(lay.segments)), P(seg)), "seg_tree")
    seg_np = seg.cpu().numpy()
    per_tensor = np.zeros(len(named_grads), dtype=np.float32)
    seen = [False] * len(named_grads)
    for i in sorted(range(len(lay.segments)), key=lambda k: (lay.segments[k].param, lay.segments[k].shard)):
        pi = lay.segments[i].param
        per_tensor[pi] = seg_np[i] if not seen[pi] else np.float32(per_tensor[pi] + seg_np[i])
        seen[pi] = True
    total = np.float32(0.0)
    for v in per_tensor:
        total = np.float32(total + v)
    return float(np.sqrt(total, dtype=np.float32)), per_tensor


def clip_grads_(named_grads: list[tuple[str, torch.Tensor]], max_norm: float, num_shards: int) -> float:
    """In-place clip of plain gradient tensors; returns the pre-clip norm. ``clip_train`` and ``clip_audit`` of the
    reference are the same function here because the trainer and the replay share one engine."""
    norm, _ = deterministic_global_norm(named_grads, num_shards)
    h = clip_coefficient(norm, max_norm)
    coef = torch.tensor(h, dtype=torch.float32)
    for _, g in named_grads:
        if g is not None:
            g.mul_(coef.to(g.device))
    return norm


clip_train = clip_grads_
clip_audit = clip_grads_
