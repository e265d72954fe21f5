"""The deterministic gradient reduction, stated on whole tensors.

The kernels (``csrc/cuda/optim_reduce.cu::grad_reduce_kernel`` and its CPU twin) apply these orders chunk by chunk inside
flat buffers; this module is the same arithmetic written out in PyTorch, for reading, for tests and for tools that want to
re-derive a reduced gradient without the engine. With V = dp_replicate x dp_shard virtual ranks, virtual rank
``r * dp_shard + s`` being shard ``s`` of replica ``r``:

    inside a replica      g_r = ((g_{r,0} + g_{r,1}) + g_{r,2}) + ...        ascending shard order, then x 1/dp_shard
    across the replicas   binary blocks: the replicas are cut into power-of-two blocks, one per set bit of the count,
                          largest first (6 = 4 + 2, 7 = 4 + 2 + 1); a block is summed as a balanced tree of adjacent pairs,
                          lower index on the left; the block sums are added left to right; then x 1/dp_replicate

fp32 addition is commutative but not associative, so this grouping is what every process count and the single-device replay
repeat. For a power-of-two count the tree is the balanced one, ((g0+g1)+(g2+g3))+...; 6 folds as ((g0+g1)+(g2+g3))+(g4+g5),
7 as (((g0+g1)+(g2+g3))+(g4+g5))+g6. ``pair_tree_sum`` is the other fixed tree of this package (strides 1, 2, 4, ...; used
over token slabs, K slabs and chunk partials, where counts are powers of two or the tail is short); the two agree while
the count has at most two set bits.
(reference src/pretrain/parallel/deterministic_reduce.py:77-117 shard fold, :140-185 binary blocks, :584-621 ``Shard(0)``)
"""
from __future__ import annotations

import torch

REPLICATE_REDUCE_ALGO = "recursive_doubling"                   # tag written into checkpoint metadata
GRAD_NORM_ALGO = "deterministic_per_tensor_sos_v1"


def binary_blocks(n: int) -> list[int]:
    """Sizes of the power-of-two blocks ``n`` items are cut into, largest first: 6 -> [4, 2], 7 -> [4, 2, 1]."""
    out, bit = [], 1 << max(n.bit_length() - 1, 0)
    while bit and n > 0:
        if n & bit:
            out.append(bit)
        bit >>= 1
    return out


def tree_reduce_sum(parts: list[torch.Tensor]) -> torch.Tensor:
    """Sum of ``parts`` in the binary-blocks order of the replica fold (module docstring). One part is returned as it is."""
    if not parts:
        raise ValueError("nothing to sum")
    total, at = None, 0
    for size in binary_blocks(len(parts)):
        level = list(parts[at:at + size])
        at += size
        while len(level) > 1:
            level = [level[i] + level[i + 1] for i in range(0, len(level), 2)]
        total = level[0] if total is None else total + level[0]
    return total


def pair_tree_sum(parts: list[torch.Tensor]) -> torch.Tensor:
    """Sum of ``parts`` by the stride tree: at stride s = 1, 2, 4, ... value k takes value k + s on its right for every k
    that is a multiple of 2s with k + s in range. Equal to ``tree_reduce_sum`` whenever ``len(parts)`` has at most two
    set bits."""
    if not parts:
        raise ValueError("nothing to sum")
    v = list(parts)
    stride = 1
    while stride < len(v):
        for k in range(0, len(v) - stride, 2 * stride):
            v[k] = v[k] + v[k + stride]
        stride *= 2
    return v[0]


def fold_virtual_ranks(grads: list[torch.Tensor], dp_shard: int, dp_replicate: int = 1) -> torch.Tensor:
    """The reduced gradient of ``V = dp_replicate * dp_shard`` virtual ranks' fp32 gradients (replica-major list): what
    ``grad_reduce_kernel`` leaves in the reduced-gradient buffer, element for element."""
    if len(grads) != dp_shard * dp_replicate:
        raise ValueError("expected %d gradients, got %d" % (dp_shard * dp_replicate, len(grads)))
    inv_s, inv_r = torch.tensor(1.0 / dp_shard, dtype=torch.float32), torch.tensor(1.0 / dp_replicate, dtype=torch.float32)
    replicas = []
    for r in range(dp_replicate):
        acc = grads[r * dp_shard].to(torch.float32)
        for s in range(1, dp_shard):
            acc = acc + grads[r * dp_shard + s].to(torch.float32)
        replicas.append(acc * inv_s)
    return tree_reduce_sum(replicas) * inv_r


def shard0_full_chunk_size(dim0: int, world_size: int) -> int:
    """Rows per shard of a ``Shard(0)`` split: ceil(dim0 / world_size)."""
    n = max(int(world_size), 1)
    return -(-int(dim0) // n)


def shard0_logical_chunk(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Rows of ``t`` that belong to shard ``rank`` (a view; fewer than the full chunk on the last shard, none past the end):
    what the sharded state hash digests."""
    size = shard0_full_chunk_size(t.shape[0], world_size)
    return t[rank * size: min((rank + 1) * size, t.shape[0])]


def shard0_chunk(t: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Shard ``rank`` padded with zero rows to the full chunk size (the shape a padded sharded tensor has everywhere)."""
    size = shard0_full_chunk_size(t.shape[0], world_size)
    rows = shard0_logical_chunk(t, rank, world_size)
    if rows.shape[0] == size:
        return rows
    pad = torch.zeros((size - rows.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    return torch.cat([rows, pad], 0) if rows.shape[0] else pad


def grad_sum_of_squares(named_grads: list[tuple[str, torch.Tensor]], num_shards: int):
    """Per-tensor sums of squares of full fp32 gradients in the canonical association (chunk partials per virtual shard,
    pair tree per segment, shards added in ascending order): a float32 array aligned with ``named_grads``."""
    from ..train.global_clip import deterministic_global_norm

    return deterministic_global_norm(named_grads, num_shards)[1]


def deterministic_total_norm(named_grads: list[tuple[str, torch.Tensor]], num_shards: int) -> float:
    """Global gradient norm with the cluster's association; identical for the trainer and the single-device replay, which
    is why one function serves both roles (the reference has ``deterministic_total_norm`` and ``audit_total_norm``,
    src/pretrain/parallel/deterministic_reduce.py:717-777)."""
    from ..train.global_clip import deterministic_global_norm

    return deterministic_global_norm(named_grads, num_shards)[0]


audit_total_norm = deterministic_total_norm

