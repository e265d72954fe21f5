"""Virtual topology arithmetic: V = dp_replicate x dp_shard virtual data-parallel ranks (replica-major),
tp ranks inside each, spread over G physical processes (reference src/pretrain/parallel/parallel_dims.py:58-194)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ParallelDims:
    dp_replicate: int
    dp_shard: int
    world_size: int          # physical processes
    tp: int = 1
    virtual_dp: int = 0      # 0 -> one virtual rank per physical dp process

    def __post_init__(self):
        if self.dp_replicate < 1 or self.tp < 1:
            raise ValueError("dp_replicate and tp must be >= 1")
        if self.world_size % self.tp:
            raise ValueError("world_size %d not divisible by tp %d" % (self.world_size, self.tp))
        dp_procs = self.world_size // self.tp
        shard = self.dp_shard
        v = self.virtual_dp or (shard if shard > 0 else max(1, dp_procs // self.dp_replicate)) * self.dp_replicate
        if shard <= 0:
            shard = v // self.dp_replicate
        if shard * self.dp_replicate != v:
            raise ValueError("virtual dp size %d != dp_replicate %d x dp_shard %d" % (v, self.dp_replicate, shard))
        if v % dp_procs:
            raise ValueError("%d virtual ranks do not split evenly over %d data-parallel processes" % (v, dp_procs))
        object.__setattr__(self, "dp_shard", shard)
        object.__setattr__(self, "virtual_dp", v)

    @property
    def dp_processes(self) -> int:
        return self.world_size // self.tp

    def hosted_virtual_ranks(self, rank: int) -> list[int]:
        per = self.virtual_dp // self.dp_processes
        dp_rank = rank // self.tp
        return list(range(dp_rank * per, (dp_rank + 1) * per))

    def coords(self, virtual_rank: int) -> tuple[int, int]:
        """(replica, shard) of a virtual rank."""
        return divmod(virtual_rank, self.dp_shard)

    def tp_rank(self, rank: int) -> int:
        return rank % self.tp

    # ---- the reference's vocabulary (src/pretrain/parallel/parallel_dims.py:141-194), answered from the virtual topology
    dp_replicate_enabled = property(lambda self: self.dp_replicate > 1)
    dp_shard_enabled = property(lambda self: self.dp_shard > 1)
    fsdp_enabled = dp_shard_enabled
    dp_enabled = property(lambda self: self.virtual_dp > 1)
    # ranks that consume distinct tokens: the VIRTUAL data-parallel size (a tensor-parallel group shares its batch)
    dp_world_size = property(lambda self: self.virtual_dp)

    def dp_rank(self, global_rank: int = 0) -> int:
        """Index of a physical rank's data-parallel process (the ranks of one tensor-parallel group share it)."""
        return global_rank // self.tp

    def make_dp_gloo_group(self):
        """A gloo group over all processes for host-side metadata (32-byte digests, scalars), or None outside a process
        group / with one process. NCCL collectives on device tensors wait for the whole stream; these do not."""
        import torch.distributed as dist

        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() <= 1:
            return None
        return dist.new_group(ranks=list(range(dist.get_world_size())), backend="gloo")

