"""Training engine: flat buffers, virtual ranks, deterministic gradient reduction, clip, AdamW.

Topology. A run is defined by its VIRTUAL data-parallel topology (V = dp_replicate x dp_shard
ranks, replica-major). The hashed arithmetic depends on that topology only. G physical processes
(GPUs, or CPU ranks) each host V / G consecutive virtual ranks and step through them in order,
which is the audit replay's virtual-rank loop (reference src/pretrain/cli/audit_replay.py:2348-2488)
used as the trainer itself; G in {1, 2, 4, 8} and the CPU replay therefore give identical bytes.

Memory (per process, sized for 180 GB HBM3e): fp32 master weights and both moments, the fp32
reduced gradient, one fp32 gradient buffer PER HOSTED VIRTUAL RANK, and the compute-dtype weights
(bf16 mixed precision; the master itself in fp32 runs). No activation recompute is needed at the
OPEN-1B micro-batch (24 GB of activations).

One optimizer step
  1. for each hosted virtual rank, for each of its micro-batches: forward + backward; weight
     gradients accumulate in fp32 straight into that rank's flat buffer (GEMM beta=1 epilogue);
  2. `grad_reduce`: every process reduces the segments it owns by reading all V buffers (its own
     and, over NVLink peer loads, the other GPUs') in ascending shard order, x 1/S, binary-blocks
     tree over replicas, x 1/R, and emits per-chunk squared-norm partials in the same pass;
  3. the partials are combined per (parameter, shard) by the pair tree, folded ascending shard then
     ascending parameter in fp32 on the host, sqrt, clip coefficient
     h = min(max_norm / (norm + 1e-6), 1)   (reference src/pretrain/train/global_clip.py:47-55);
  4. `adamw_push`: g *= h, decoupled-decay AdamW on the owned segments, and the new weights are
     stored, in compute dtype, into the weight buffer of EVERY GPU (the parameter all-gather done
     by peer stores from inside the update kernel).
On CPU ranks (gloo) the gradient buffers are exchanged with all_gather and every rank applies the
identical update to all segments.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from ..config.schema import RootConfig
from ..models import build_model, fused_ce_z_loss, init_weights, streaming_head_loss
from ..models.modules.core import refresh_lsq_weight_scales, set_qat_active
from ..models.precision import PrecisionPolicy
from ..ops import functional as K
from ..ops.autograd import GradSlot, set_tp, wgrad_join
from ..ops.native import F, I, P, check, cpu_lib, cuda_lib, stream_ptr
from ..parallel.flat import FlatLayout, PeerBuffer, lazy_zeros
from ..parallel.parallel_dims import ParallelDims
from . import state_hash as SH


@dataclass
class StepOutput:
    ce_per_vrank: dict          # virtual rank -> list of per-micro-batch CE (python floats)
    z_per_vrank: dict
    grad_norm: float
    clip_coef: float
    skipped: bool


_OFFLOAD_BLOCK = 1 << 26  # elements per copy between a state file and the GPU (256 MiB of fp32)


class SpillCorruption(RuntimeError):
    """A gradient partial read back from disk does not match the digest written with it."""


def build_param_groups(named_params, no_decay_names, lr, betas, eps, weight_decay):
    """[decay, no_decay] groups: a parameter is not decayed if it has fewer than 2 dims or its name contains
    one of ``no_decay_names`` (reference src/pretrain/optim/adamw.py:21-63). Returns (groups, membership)."""
    member = []
    for name, p in named_params:
        member.append(1 if (p.dim() < 2 or any(s in name for s in no_decay_names)) else 0)
    base = dict(lr=float(lr), betas=[float(betas[0]), float(betas[1])], eps=float(eps), amsgrad=False)
    groups = [dict(base, name="decay", weight_decay=float(weight_decay)), dict(base, name="no_decay", weight_decay=0.0)]
    return groups, member


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class TrainEngine:
    def __init__(self, cfg: RootConfig, device: torch.device | str = "cpu", rank: int = 0, world: int = 1, group=None,
                 seed: int | None = None, init: bool = True, fold_gradients: bool = False, fold_spill_dir: str | None = None,
                 offload_optimizer: bool = False, optimizer_offload_dir: str | None = None,
                 offload_master: bool = False, master_offload_dir: str | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.rank, self.world, self.group = rank, world, group
        run = cfg.run
        # virtual topology arithmetic (V = dp_replicate x dp_shard virtual ranks; ``tp`` consecutive processes form a group
        # that works on each micro-batch together; the ``dp_groups`` groups share the virtual ranks between them)
        dims = ParallelDims(max(1, run.dp_replicate_size), run.dp_shard_size, world, max(1, int(run.tp_size)), max(0, run.virtual_dp_size))
        self.dims = dims
        self.dp_replicate, self.dp_shard, self.V, self.tp = dims.dp_replicate, dims.dp_shard, dims.virtual_dp, dims.tp
        self.dp_groups, self.dp_rank, self.tp_rank = dims.dp_processes, rank // dims.tp, dims.tp_rank(rank)
        self.hosted = dims.hosted_virtual_ranks(rank)
        # Small host-side exchanges (digests, batch chains, logged scalars) go over a gloo group of their own: a library
        # collective on device tensors would first wait for everything queued on the stream - the whole backward pass - and
        # stall the host that should be queueing the next kernels. CPU ranks already talk gloo.
        self.host_group = group
        if world > 1 and group is None and dist.get_backend() != "gloo":
            self.host_group = dist.new_group(backend="gloo")
        self._host_gloo = world > 1 and dist.get_backend(self.host_group) == "gloo"
        self._tp_state = None
        if self.tp > 1:
            from ..ops.autograd import TpState

            tp_group = group
            if self.dp_groups > 1:  # every process creates every group, in the same order
                tp_group = None
                for d in range(self.dp_groups):
                    g_ = dist.new_group([d * self.tp + t for t in range(self.tp)])
                    if d == self.dp_rank:
                        tp_group = g_
            self._tp_state = TpState(tp_group, self.tp_rank, self.tp)
            self._tp_group = tp_group
        self.mixed = bool(run.mixed_precision)
        self.precision = PrecisionPolicy.from_run(self.mixed)
        self.compute_dtype = self.precision.param_dtype
        self.is_cuda = self.device.type == "cuda"
        if self.tp > 1 and run.tp_fused and self.is_cuda and self.mixed:
            if run.activation_checkpoint:
                raise ValueError("run.tp_fused keeps each layer's gathered activation in its peer buffer; it is not combined with activation checkpointing")
            from ..parallel.tensor_parallel import TpWorkspace

            self._tp_state.ws = TpWorkspace(self.device, self.tp_rank, self.tp, self._tp_group)
        self.lib = cuda_lib() if self.is_cuda else cpu_lib()
        # ``run.parallel: ddp`` (replicated parameters, library all-reduce of the gradients; reference src/pretrain/parallel/fsdp.py:24-54)
        # is the throughput-only mode here as well: same path as ``reduction_mode: nccl``, order not pinned, not auditable
        self.nccl_mode = run.reduction_mode == "nccl" or run.parallel == "ddp"

        # ---- model on the meta device first: the layout decides where the parameters live
        model = build_model(cfg.model)
        model.compute_dtype = self.compute_dtype
        model.activation_checkpoint = bool(run.activation_checkpoint)
        model.ac_every_other_block = bool(run.ac_every_other_block)
        named = list(model.named_parameters())
        self.param_groups, member = build_param_groups(named, cfg.optim.no_decay_param_names, cfg.optim.peak_lr, cfg.optim.betas,
                                                       cfg.optim.eps, cfg.optim.weight_decay)
        self.layout = FlatLayout.build([(n, tuple(p.shape)) for n, p in named], self.dp_shard, member)
        lay = self.layout
        n = lay.total
        # Tensor-parallel groups on GPUs of one machine keep the sharded ownership too: every process of the run owns a run of
        # segments, and the reduction kernel assembles each virtual rank's gradient from the disjoint slices its tensor-
        # parallel ranks wrote (integer sum of bit patterns) while it pulls them. Elsewhere (CPU ranks, several machines) a
        # tensor-parallel run assembles by an integer all-reduce and every process reduces and updates everything itself.
        # How the gradient buffers of the other processes are reached (OTB_GRAD_TRANSPORT = auto | peer | collective | gather):
        #   peer       - sharded ownership, plain loads from the other GPUs' buffers (CUDA IPC over NVLink; one machine);
        #   collective - sharded ownership, every process SENDS each owner its segments (point-to-point messages of the
        #                process group: NCCL between machines, gloo on CPU ranks), the owner reduces its own copies with
        #                the same kernel and the updated weights come back by all-gather;
        #   gather     - every process gathers whole buffers and reduces everything itself (small models, CPU tests,
        #                tensor-parallel groups).
        # ``auto``: GPUs of one machine -> peer, GPUs of several machines -> collective, CPU ranks -> gather.
        transport = os.environ.get("OTB_GRAD_TRANSPORT", "auto")
        if transport not in ("auto", "peer", "collective", "gather"):
            raise ValueError("OTB_GRAD_TRANSPORT=%s (auto, peer, collective or gather)" % transport)
        can_shard = world > 1 and not self.nccl_mode and (self.tp == 1 or (self.is_cuda and transport in ("auto", "peer")))
        if transport == "auto":
            transport = "gather"
            if can_shard and self.is_cuda:
                import socket

                hosts: list = [None] * world
                dist.all_gather_object(hosts, socket.gethostname(), group=group)
                transport = "peer" if len(set(hosts)) == 1 else "collective"
        if not can_shard or (self.tp > 1 and transport != "peer"):
            transport = "gather"
        if transport == "peer" and not self.is_cuda:
            raise ValueError("OTB_GRAD_TRANSPORT=peer needs GPUs (peer loads over NVLink)")
        self.transport = transport
        if world > 1 and rank == 0:
            import logging

            logging.getLogger(__name__).info("gradient transport: %s (%d processes, tensor-parallel groups of %d)", transport, world, self.tp)
        peer = transport == "peer"
        self.collective = transport == "collective"
        self.sharded = peer or self.collective
        pw, pg = (rank, world) if peer else (0, 1)

        def alloc(nbytes, shared):
            return PeerBuffer(nbytes, self.device, pw if shared else 0, pg if shared else 1, group if shared else None)

        # State kept off the compute device between steps (single-process replay of a model whose training state does
        # not fit beside the activations). Moments: on the CPU the two flat buffers ARE file mappings in
        # ``optimizer_offload_dir`` (the kernels work on them in place and ``release_state`` lets the OS drop the pages);
        # on a GPU they are written to those files after the step's hash and read back for the next optimizer step, so
        # they are absent during forward and backward, when the activations peak. Master weights: file mapping on the
        # CPU; on a GPU they stay resident (the parameters are views of that buffer).
        # (reference: --offload-optimizer / --offload-master, src/pretrain/cli/audit_replay.py:1249-1290)
        self._off_opt, self._off_master = bool(offload_optimizer), bool(offload_master)
        if (self._off_opt or self._off_master) and (world != 1 or self.tp != 1):
            raise ValueError("state offload is for the single-process replay")
        self._off_tmp = []
        self._off_files: dict[str, np.memmap] = {}
        self.master_offload_inert = self._off_master and self.is_cuda
        if self._off_master and not self.is_cuda:
            backing = torch.from_numpy(self._mapped_file("master", master_offload_dir, 4 * n, np.uint8))
            self.buf_master = PeerBuffer(4 * n, self.device, storage=backing)
        else:
            self.buf_master = alloc(4 * n, shared=not self.mixed)
        self.master = self.buf_master.typed(torch.float32)
        if self.mixed:
            self.buf_compute = alloc(2 * n, shared=True)
            self.compute = self.buf_compute.typed(torch.bfloat16)
        else:
            self.buf_compute, self.compute = self.buf_master, self.master
        # (the moments and the reduced gradient are allocated below, once the ownership is known)
        # Folded gradients (single-process replay with little memory): instead of one gradient buffer per hosted virtual
        # rank there is ONE work buffer plus one partial per replica; ``fold_virtual_rank`` adds a finished virtual rank
        # into its replica's partial in ascending shard order - the same left fold, element by element, that the reduction
        # kernel runs over separate buffers - and a finished partial may be spilled to disk with a digest beside it.
        # Streaming vocabulary head (exact fp32 family only, where a weight gradient accumulated panel by panel is the
        # same sequential chain as the unstreamed one): PRETRAIN_AUDIT_STREAM_HEAD=1, or the ``stream_head`` attribute.
        # (reference src/pretrain/model/streaming_head_loss.py:15-118, used by src/pretrain/cli/audit_replay.py:2312)
        self.stream_head = os.environ.get("PRETRAIN_AUDIT_STREAM_HEAD") == "1" and not self.mixed and self.tp == 1
        self._phase: list | None = [] if os.environ.get("PRETRAIN_CUDA_EVENT_TIMING") == "1" else None
        self.fold = bool(fold_gradients)
        if self.fold and (world != 1 or self.tp != 1):
            raise ValueError("folded gradients are for the single-process replay")
        self._fold_spill = fold_spill_dir
        self._partials: dict[int, object] = {}   # replica -> fp32 tensor, or the path it was spilled to
        self.buf_grads = [alloc(4 * n, shared=True) for _ in (self.hosted[:1] if self.fold else self.hosted)]
        self.grads = [b.typed(torch.float32) for b in self.buf_grads]
        for g in self.grads:
            g.zero_()
        self._stale = [False] * len(self.grads)
        self.opt_step = 0
        self.global_step = None  # set by the loop / the replay: QAT gates follow the run's step, not the optimizer's

        # ---- chunk tables on the device, ownership
        dev = self.device
        self.chunk_start = torch.from_numpy(lay.chunk_start).to(dev)
        self.chunk_len = torch.from_numpy(lay.chunk_len).to(dev)
        self.chunk_group = torch.from_numpy(lay.chunk_group).to(dev)
        self.seg_first = torch.from_numpy(lay.seg_first).to(dev)
        self.n_chunks = len(lay.chunk_start)
        self.n_segs = len(lay.segments)
        if self.sharded:
            ranges = lay.owner_ranges(world)
        else:
            ranges = [(0, self.n_segs)] * world
        self.seg_lo, self.seg_hi = ranges[rank]
        self.chunk_lo = int(lay.seg_first[self.seg_lo])
        self.chunk_hi = int(lay.seg_first[self.seg_hi])
        self.peer = peer
        # Packed layout of every owner's segments (each starting at a multiple of 64 elements): what travels in the
        # point-to-point transport, and where the moments and the reduced gradient live when the state is sharded
        self._packed_state = bool(self.sharded and (run.state_sharding or os.environ.get("OTB_STATE_SHARDING") == "1"))
        self._pack_off, self._pack_len, self._owner_ranges = [], [], ranges
        if self.sharded:
            for slo, shi in ranges:
                offs, off = [], 0
                for sg in lay.segments[slo:shi]:
                    offs.append(off)
                    off += -(-sg.length // 64) * 64
                self._pack_off.append(offs)
                self._pack_len.append(max(off, 64))
        n_state = self._pack_len[rank] if self._packed_state else n
        self.chunk_state_start = None
        if self._packed_state:
            st = np.full(len(lay.chunk_start), -1, dtype=np.int64)
            for sg, off in zip(lay.segments[self.seg_lo:self.seg_hi], self._pack_off[rank]):
                for c in range(sg.first_chunk, sg.first_chunk + sg.n_chunks):
                    st[c] = off + int(lay.chunk_start[c]) - sg.start
            self.chunk_state_start = torch.from_numpy(st).to(dev)
        if self._off_opt:
            for key in ("exp_avg", "exp_avg_sq"):
                self._mapped_file(key, optimizer_offload_dir, n, np.float32)
        if self._off_opt and not self.is_cuda:
            self._m1 = torch.from_numpy(self._off_files["exp_avg"])
            self._m2 = torch.from_numpy(self._off_files["exp_avg_sq"])
        else:
            self._m1 = torch.zeros(n_state, dtype=torch.float32, device=self.device)
            self._m2 = torch.zeros(n_state, dtype=torch.float32, device=self.device)
        self.grad_red = lazy_zeros(n_state, torch.float32, self.device)
        if self.collective:
            # the chunk table of this process's own segments inside its packed buffer
            mine = []
            for sg, off in zip(lay.segments[self.seg_lo:self.seg_hi], self._pack_off[rank]):
                for c in range(sg.first_chunk, sg.first_chunk + sg.n_chunks):
                    mine.append(off + int(lay.chunk_start[c]) - sg.start)
            self._packed_chunk_start = torch.from_numpy(np.asarray(mine, dtype=np.int64)).to(dev)
        # ``optim.name: muon_hybrid`` (experimental, outside the audited path): Muon on the 2-D block weights, the AdamW
        # kernel on everything else through a chunk table without those parameters
        # (reference src/pretrain/optim/muon.py:24-164, gated by config in src/pretrain/optim/registry.py:13-27)
        self.muon_params: list[int] = []
        if cfg.optim.name == "muon_hybrid":
            if self.sharded or self.tp > 1:
                raise NotImplementedError("optim.name=muon_hybrid needs every process to hold whole gradients: one GPU, CPU ranks, "
                                          "or run.reduction_mode=nccl")
            from ..optim.muon import is_hidden_matrix

            self.muon_params = [i for i, (nm, shp) in enumerate(zip(lay.names, lay.shapes)) if is_hidden_matrix(nm, shp)]
            hidden = set(self.muon_params)
            keep = np.concatenate([np.arange(sg.first_chunk, sg.first_chunk + sg.n_chunks) for sg in lay.segments if sg.param not in hidden]
                                  or [np.zeros(0, dtype=np.int64)]).astype(np.int64)
            self._aux_chunks = (torch.from_numpy(lay.chunk_start[keep]).to(dev), torch.from_numpy(lay.chunk_len[keep]).to(dev),
                                torch.from_numpy(lay.chunk_group[keep]).to(dev), int(len(keep)))
        self.chunk_sos = torch.zeros(max(self.n_chunks, 1), dtype=torch.float32, device=dev)
        self.seg_sos = torch.zeros(max(self.n_segs, 1), dtype=torch.float32, device=dev)
        self._setup_overlap()

        # ---- initialise (CPU-sampled Philox, byte-copied) and move the model onto the flat buffers
        if init:
            if self.is_cuda:
                # the sampling runs on the host whatever the device: give it this process's share of the cores even where
                # the launcher pinned OMP_NUM_THREADS to 1 (same bytes at any thread count)
                from ..ops.native import host_threads

                with host_threads():
                    init_weights(model, cfg.run.seed if seed is None else seed)
            else:
                # on the host the parameters become views of the master buffer BEFORE they are sampled, so that the stream
                # is written once, where it will live (no second copy of the model, no second pass over its pages)
                for i, (name, p) in enumerate(named):
                    if p.dtype == torch.float32:
                        p.data = lay.view(self.master, i)
                init_weights(model, cfg.run.seed if seed is None else seed)
        with torch.no_grad():
            for i, (name, p) in enumerate(named):
                dst = lay.view(self.master, i)
                if p.data_ptr() != dst.data_ptr():
                    dst.copy_(p.detach().to(torch.float32))
        self.model = model
        self.names = lay.names
        self.slots = [GradSlot() for _ in named]
        self._install_views()
        self._setup_param_gather()
        self.refresh_compute_weights()
        # buffers (RoPE tables) follow the device
        for mod in self.model.modules():
            for bname, b in list(mod.named_buffers(recurse=False)):
                mod._buffers[bname] = b.to(self.device)

    # ------------------------------------------------------- parameter all-gather inside the consuming GEMM
    def _setup_param_gather(self) -> None:
        """``run.param_sharding: gather`` (or OTB_PARAM_SHARDING=gather): the AdamW kernel keeps the new bf16 rows of the
        projection weights on the owner, and the first forward GEMM after an update pulls the other owners' rows itself
        (parallel/param_gather.py; kernel otb_pg_gemm). Embedding, norm gains and any weight whose rows are not split
        evenly over the processes are still pushed to every GPU by the AdamW kernel."""
        self._pg = None
        mode = os.environ.get("OTB_PARAM_SHARDING") or self.cfg.run.param_sharding
        if mode != "gather" or self.world == 1:  # one process owns every row: nothing to gather (the replay of such a run)
            return
        if not (self.is_cuda and self.peer and self.sharded and self.mixed and self.tp == 1) or self.cfg.model.qat.enabled or self.muon_params:
            raise ValueError("run.param_sharding=gather needs GPUs of one machine with sharded ownership over peer memory, bf16 compute "
                             "weights, AdamW, no tensor parallelism and no quantisation-aware training")
        from ..models.modules.core import Linear
        from ..parallel.param_gather import GatheredWeight, flag_words, uniform_rows_per_owner

        lay = self.layout
        modules = dict(self.model.named_modules())
        idx = {n: i for i, n in enumerate(lay.names)}

        def rows_per_owner(i: int) -> int | None:
            shape = lay.shapes[i]
            row = lay.numels[i] // shape[0]
            ranges = []
            for slo, shi in self._owner_ranges:
                segs = sorted((sg for sg in lay.segments[slo:shi] if sg.param == i), key=lambda g: g.start)
                if not segs:
                    ranges.append((0, 0))
                    continue
                if any(a.start + a.length != b.start for a, b in zip(segs, segs[1:])):
                    return None
                lo = (segs[0].start - lay.offsets[i]) // row
                ranges.append((lo, lo + sum(g.length for g in segs) // row))
            return uniform_rows_per_owner(ranges, shape[0])

        groups = []   # (slot, parameter indices, element offset of row 0, rows, cols)
        fused = set()
        for slot, o0, rows, cols, members in self._fused:
            groups.append((slot, tuple(members), o0, rows, cols))
            fused.update(members)
        for name, i in idx.items():
            mod_name, _, attr = name.rpartition(".")
            mod = modules[mod_name]
            if i in fused or attr != "weight" or type(mod) is not Linear or len(lay.shapes[i]) != 2:
                continue
            groups.append((self.slots[i], (i,), lay.offsets[i], lay.shapes[i][0], lay.shapes[i][1]))
        weights, pulled, blocks = [], set(), 0
        plans = []
        for slot, members, o0, rows, cols in groups:
            rpo = [rows_per_owner(i) for i in members]
            if any(r is None for r in rpo) or cols % 8 or (2 * o0) % 16:
                continue
            begins, at = [], 0
            for i in members:
                begins.append(at)
                at += lay.shapes[i][0]
            plans.append((slot, members, o0, rows, cols, begins, rpo, blocks))
            blocks += flag_words(rows)
        self._pg_flags = torch.zeros(max(blocks, 1), dtype=torch.int32, device=self.device)
        for slot, members, o0, rows, cols, begins, rpo, b0 in plans:
            local = self.compute[o0:o0 + rows * cols].view(rows, cols)
            gw = GatheredWeight(local, [p + 2 * o0 for p in self.buf_compute.ptrs], self.rank, begins, rpo,
                                self._pg_flags[b0:b0 + flag_words(rows)])
            slot.gather = gw
            weights.append(gw)
            pulled.update(members)
        # the owned chunks, split into those of pulled weights (stored locally by the AdamW kernel) and the rest (pushed)
        own = np.arange(self.chunk_lo, self.chunk_hi, dtype=np.int64)
        chunk_param = np.zeros(len(lay.chunk_start), dtype=np.int64)
        for sg in lay.segments:
            chunk_param[sg.first_chunk:sg.first_chunk + sg.n_chunks] = sg.param
        is_pull = np.isin(chunk_param[own], np.fromiter(pulled, dtype=np.int64, count=len(pulled)))
        tables = {}
        for key, ids in (("pull", own[is_pull]), ("push", own[~is_pull])):
            t = torch.from_numpy(ids).to(self.device)
            tables[key] = (self.chunk_start[t].contiguous(), self.chunk_len[t].contiguous(), self.chunk_group[t].contiguous(),
                           None if self.chunk_state_start is None else self.chunk_state_start[t].contiguous(), int(len(ids)))
        self._pg = {"weights": weights, "tables": tables, "epoch": 0, "pulled_params": sorted(pulled)}

    def complete_compute_weights(self) -> None:
        """Gather mode: make every GPU's bf16 weights whole NOW (each owner pushes the rows it kept back), for readers
        that are not a forward GEMM - weight statistics, an evaluation outside the step. Every process calls it."""
        if self._pg is None or not any(g.pending() for g in self._pg["weights"]):
            return
        cs, cl, _cg, _sst, cnt = self._pg["tables"]["pull"]
        if cnt:
            check(self.lib.otb_push_cast(P(cs), P(cl), I(cnt), P(self.master), _ptr_array(self.buf_compute.ptrs), I(len(self.buf_compute.ptrs)),
                                         I(1), stream_ptr()), "push_cast")
        self._stream_barrier()
        for g in self._pg["weights"]:
            g.mark_complete()

    # ------------------------------------------------------- gradient reduction under the backward pass
    def _setup_overlap(self) -> None:
        """Bucketed reduction that runs under the backward pass of the step's last micro-batch on this process.

        The reference starts its reduce-scatter from inside the last micro-batch's backward, one FSDP module at a time
        (src/pretrain/train/loop.py:872-873, 904; src/pretrain/parallel/deterministic_reduce.py:504-523). Here a bucket is
        the vocabulary head, one transformer block (the final norm goes with the last block), or the embedding. When the
        backward pass has finished a bucket (`BucketMarkFn`), this process
          1. tells every peer so: one release store of the step's epoch into word [bucket, rank] of each GPU's flag array,
          2. queues, on a side stream, a bounded wait for the same word of every rank followed by the reduction kernel
             over the chunks of that bucket which this process owns.
        The peers' gradients of block L thus cross NVLink while blocks < L are still in their backward pass. The kernel, the
        chunk table and therefore every sum are those of the one-shot reduction: only the launch granularity changes.
        OTB_REDUCE_OVERLAP = auto (GPUs: on) | 1 (also on the CPU, where it runs synchronously: tests) | 0."""
        self._ov = None
        mode = os.environ.get("OTB_REDUCE_OVERLAP", "auto")
        eligible = (self.tp == 1 and not self.fold and not self.nccl_mode and not self.collective and not self.stream_head
                    and not self.muon_params and (self.peer or self.world == 1))
        if not eligible or mode == "0" or (mode == "auto" and not self.is_cuda):
            return
        lay, L = self.layout, self.cfg.model.n_layers

        def bucket_of(name: str) -> int:  # in the order in which the backward pass completes them
            if name.startswith("embedding.output."):
                return 0
            if name.startswith("norm_out."):
                return 1
            if name.startswith("blocks."):
                return 1 + (L - 1 - int(name.split(".")[1]))
            return L + 1  # token embedding and the norm on its output: the end of the backward pass

        ids: list[list[int]] = [[] for _ in range(L + 2)]
        for sg in lay.segments[self.seg_lo:self.seg_hi]:
            ids[bucket_of(lay.names[sg.param])].extend(range(sg.first_chunk, sg.first_chunk + sg.n_chunks))
        per = self.V // self.dp_groups
        srcs = []
        for v in range(self.V):
            r, slot = v // per, v % per
            srcs.append(self.buf_grads[slot].ptrs[r] if self.peer else self.grads[slot].data_ptr())
        ov = {"ids": [torch.tensor(x, dtype=torch.int32, device=self.device) for x in ids], "n": [len(x) for x in ids],
              "srcs": _ptr_array(srcs), "epoch": 0, "active": False, "launched": set(), "unwritten": None,
              "budget_ns": int(float(os.environ.get("OTB_PEER_WAIT_MS", "30000")) * 1e6),
              # OTB_REDUCE_TIMELINE=1: CUDA events per bucket (ready / reduction start / reduction end), see overlap_timeline()
              "timeline": [] if os.environ.get("OTB_REDUCE_TIMELINE") == "1" else None}
        if self.is_cuda:
            ov["reduce_stream"] = torch.cuda.Stream(device=self.device)
            ov["signal_stream"] = torch.cuda.Stream(device=self.device)
        if self.peer:
            ov["flags"] = PeerBuffer(4 * (L + 2) * self.world, self.device, self.rank, self.world, self.group)
            ov["bar"] = PeerBuffer(4 * 8, self.device, self.rank, self.world, self.group)
            ov["bar_seq"] = 0
        self._ov = ov

    def _block_done(self, block: int) -> None:
        """Called from the backward pass (models/llama3.py): block `block` and everything after it are done; -1 = the head."""
        L = self.cfg.model.n_layers
        self._launch_bucket(0 if block < 0 else 1 + (L - 1 - block))

    def _launch_bucket(self, b: int) -> None:
        ov = self._ov
        if b in ov["launched"]:
            return
        ov["launched"].add(b)
        S, R = self.dp_shard, self.dp_replicate
        if not self.is_cuda:
            if ov["n"][b]:
                check(self.lib.otb_cpu_grad_reduce_ex(ov["srcs"], I(S), I(R), P(self.chunk_start), P(self.chunk_len), P(ov["ids"][b]),
                                                      I(ov["n"][b]), P(self.chunk_state_start), P(self.grad_red), P(self.chunk_sos)), "grad_reduce_ids")
            return
        wgrad_join()
        timed = ov["timeline"] is not None
        done = torch.cuda.Event(enable_timing=timed)
        done.record()  # everything the backward pass has queued for this bucket
        red = ov["reduce_stream"]
        if self.peer:
            sig = ov["signal_stream"]
            sig.wait_event(done)
            check(self.lib.otb_flag_signal(_ptr_array(ov["flags"].ptrs), I(self.world), I(b * self.world + self.rank),
                                           ctypes.c_uint(ov["epoch"]), ctypes.c_void_p(sig.cuda_stream)), "flag_signal")
        red.wait_event(done)
        pending = getattr(self, "_hash_done", None)
        if pending is not None:
            red.wait_event(pending)  # the previous step's digests still read the reduced gradient
        rs = ctypes.c_void_p(red.cuda_stream)
        if self.peer:
            check(self.lib.otb_flag_wait(ctypes.c_void_p(ov["flags"].ptrs[self.rank]), I(b * self.world), I(self.world),
                                         ctypes.c_uint(ov["epoch"]), ctypes.c_ulonglong(ov["budget_ns"]), P(K._status(self.device)),
                                         ctypes.c_uint(4), rs), "flag_wait")
        if timed:
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record(red)
        if ov["n"][b]:
            check(self.lib.otb_grad_reduce_ex(ov["srcs"], I(S), I(R), I(1), P(self.chunk_start), P(self.chunk_len), P(ov["ids"][b]),
                                              I(ov["n"][b]), P(self.chunk_state_start), P(self.grad_red), P(self.chunk_sos), rs), "grad_reduce_ids")
        if timed:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(red)
            ov["timeline"].append((ov["epoch"], b, done, t0, t1))

    def overlap_timeline(self) -> list[dict]:
        """With OTB_REDUCE_TIMELINE=1: for every bucket of the last overlapped step, when the backward pass finished it,
        when its reduction began (all ranks had signalled) and ended, in ms after the first bucket became ready, plus
        `backward_end_ms`, the moment the backward pass itself was done. One device synchronisation."""
        ov = self._ov
        if ov is None or not ov.get("timeline"):
            return []
        torch.cuda.synchronize()
        rows = [r for r in ov["timeline"] if r[0] == ov["epoch"]]
        base = rows[0][2]
        end = getattr(self, "_bwd_end_event", None)
        out = [{"bucket": b, "chunks": ov["n"][b], "ready_ms": base.elapsed_time(d), "reduce_start_ms": base.elapsed_time(t0),
                "reduce_end_ms": base.elapsed_time(t1)} for _, b, d, t0, t1 in rows]
        if end is not None:
            for r in out:
                r["backward_end_ms"] = base.elapsed_time(end)
        ov["timeline"].clear()
        return out

    def _stream_barrier(self) -> None:
        """All processes have reached this point of their streams (flag exchange over peer memory on the current stream;
        bounded wait, no host synchronisation). Falls back to the host barrier where there is no peer memory."""
        ov = self._ov
        if ov is None or not self.peer:
            self._barrier()
            return
        ov["bar_seq"] += 1
        check(self.lib.otb_peer_barrier(_ptr_array(ov["bar"].ptrs), I(self.rank), I(self.world), ctypes.c_uint(ov["bar_seq"]),
                                        P(K._status(self.device)), stream_ptr()), "peer_barrier")

    # ------------------------------------------------------------------------------ phase timing
    def _tick(self, phase: str | None):
        """Phase timers (PRETRAIN_CUDA_EVENT_TIMING=1): a CUDA event on the current stream (a host clock on the CPU) at
        every phase boundary; ``phase`` names the interval that ENDS here (None opens one). Nothing is synchronised
        until ``phase_report`` (reference src/pretrain/train/loop.py:733-743, 875-909, 1036-1051)."""
        if self._phase is None:
            return
        if self.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
        else:
            import time

            ev = time.perf_counter()
        self._phase.append((phase, ev))

    def phase_report(self) -> dict:
        """{"phase_fwd_ms", "phase_bwd_ms", "phase_clip_ms", "phase_opt_ms"} since the last report (one synchronise)."""
        out: dict[str, float] = {}
        if not self._phase:
            return out
        if self.is_cuda:
            self._phase[-1][1].synchronize()
        for (_, a), (name, b) in zip(self._phase[:-1], self._phase[1:]):
            if name is not None:
                ms = a.elapsed_time(b) if self.is_cuda else (b - a) * 1e3
                out["phase_%s_ms" % name] = out.get("phase_%s_ms" % name, 0.0) + ms
        self._phase = []
        return out

    # ------------------------------------------------------------------------------ state offload
    def _mapped_file(self, key: str, directory: str | None, count: int, dtype) -> np.memmap:
        """A zero-filled file mapping of ``count`` elements in ``directory`` (a temporary directory when None)."""
        import tempfile

        if directory is None:
            tmp = tempfile.TemporaryDirectory(prefix="otb_offload_")
            self._off_tmp.append(tmp)
            directory = tmp.name
        os.makedirs(directory, exist_ok=True)
        mm = np.memmap(os.path.join(directory, key + ".bin"), dtype=dtype, mode="w+", shape=(max(int(count), 1),))
        self._off_files[key] = mm
        return mm

    def _moments_in(self) -> None:
        if self._m1 is None:  # GPU, released: read the two files back
            for attr, key in (("_m1", "exp_avg"), ("_m2", "exp_avg_sq")):
                t = torch.empty(self.layout.total, dtype=torch.float32, device=self.device)
                src = self._off_files[key]
                for lo in range(0, t.numel(), _OFFLOAD_BLOCK):
                    hi = min(lo + _OFFLOAD_BLOCK, t.numel())
                    t[lo:hi].copy_(torch.from_numpy(src[lo:hi]))
                setattr(self, attr, t)

    @property
    def m1(self) -> torch.Tensor:
        self._moments_in()
        return self._m1

    @property
    def m2(self) -> torch.Tensor:
        self._moments_in()
        return self._m2

    def release_state(self) -> None:
        """Between two steps of a replay with offloaded state: after the step's hash, before the next forward. Moments
        leave the GPU (written to their files) or, on the CPU, their pages are handed back to the OS; the same for a
        file-mapped master copy when a separate compute copy serves forward and backward. No value changes."""
        if not (self._off_opt or self._off_master):
            return
        import mmap

        if self.is_cuda:
            self._wait_pending_hash()
            torch.cuda.synchronize()
        if self._off_opt and self.is_cuda and self._m1 is not None:
            for attr, key in (("_m1", "exp_avg"), ("_m2", "exp_avg_sq")):
                t, dst = getattr(self, attr), self._off_files[key]
                for lo in range(0, t.numel(), _OFFLOAD_BLOCK):
                    hi = min(lo + _OFFLOAD_BLOCK, t.numel())
                    dst[lo:hi] = t[lo:hi].cpu().numpy()
                setattr(self, attr, None)
            self.__dict__.pop("_hash_plans", None)  # the digest plans hold the freed addresses
            torch.cuda.empty_cache()
        drop = []
        if self._off_opt:
            drop += ["exp_avg", "exp_avg_sq"]
        if self._off_master and not self.is_cuda and self.mixed:
            drop.append("master")
        for key in drop:
            mm = self._off_files[key]
            mm.flush()
            try:
                mm._mmap.madvise(mmap.MADV_DONTNEED)  # a shared file mapping: the data stays in the file
            except (AttributeError, OSError, ValueError):
                pass

    # ------------------------------------------------------------------------------ plumbing
    def _install_views(self) -> None:
        lay = self.layout
        byname = dict(self.model.named_parameters())
        modules = dict(self.model.named_modules())
        for i, name in enumerate(lay.names):
            p = byname[name]
            p.data = lay.view(self.master, i)
            mod_name, _, attr = name.rpartition(".")
            mod = modules[mod_name]
            setattr(mod, "_compute_" + attr, lay.view(self.compute, i))
            setattr(mod, "_slot_" + attr, self.slots[i])
        # fused QKV: wq|wk|wv are adjacent in the flat buffers
        idx = {n: i for i, n in enumerate(lay.names)}
        self._fused = []
        for mname, mod in modules.items():
            if all(hasattr(mod, a) for a in ("wq", "wk", "wv")):
                iq, ik, iv = (idx["%s.%s.weight" % (mname, a)] for a in ("wq", "wk", "wv"))
                o0 = lay.offsets[iq]
                contiguous = lay.offsets[ik] == o0 + lay.numels[iq] and lay.offsets[iv] == lay.offsets[ik] + lay.numels[ik]
                if not contiguous:
                    continue
                rows = lay.shapes[iq][0] + lay.shapes[ik][0] + lay.shapes[iv][0]
                cols = lay.shapes[iq][1]
                slot = GradSlot()
                compute_v = self.compute[o0:o0 + rows * cols].view(rows, cols)
                mod._fused_qkv = (byname["%s.wq.weight" % mname], compute_v, slot)
                self._fused.append((slot, o0, rows, cols, (iq, ik, iv)))

    def _bind_slots(self, gbuf: torch.Tensor | None, fresh: bool = False) -> None:
        """Point every gradient slot at its view of ``gbuf``. ``fresh``: the buffer holds last step's values, so the
        first writer of each slot stores instead of accumulating (see ``GradSlot``)."""
        lay = self.layout
        for i, slot in enumerate(self.slots):
            slot.buf = None if gbuf is None else lay.view(gbuf, i)
            slot.fresh, slot.written = fresh, False
        for slot, o0, rows, cols, _members in self._fused:
            slot.buf = None if gbuf is None else gbuf[o0:o0 + rows * cols].view(rows, cols)
            slot.fresh, slot.written = fresh, False

    def _zero_unwritten_slots(self) -> set:
        """After the first backward pass into a stale buffer: parameters nobody wrote get an explicit zero."""
        covered = set()
        for slot, _o0, _rows, _cols, members in self._fused:
            if slot.written:
                covered.update(members)
        unwritten = set()
        for i, slot in enumerate(self.slots):
            if not slot.written and i not in covered and slot.buf is not None:
                slot.buf.zero_()
                unwritten.add(i)
        return unwritten

    def named_master(self):
        return [(n, self.layout.view(self.master, i)) for i, n in enumerate(self.names)]

    def resident_bytes(self) -> dict:
        """Bytes of training state this process holds, by kind (activations and collective staging excluded)."""
        n = self.layout.total
        ns = self._pack_len[self.rank] if self._packed_state else n  # moments and reduced gradient: owned segments only when sharded
        out = {"master": 4 * n, "moments": 0 if (self._off_opt and self._m1 is None) else 8 * ns, "reduced_gradient": 4 * ns,
               "gradient_buffers": 4 * n * len(self.grads), "compute_weights": 2 * n if self.mixed else 0}
        out["total"] = sum(out.values())
        return out

    def named_weights_for_stats(self):
        """Complete current weights for telemetry: the fp32 master where this process holds all of it, else the compute
        copy (with peer-sharded ownership only the owned segments of the master are current; the compute copy is whole)."""
        src = self.compute if self.sharded else self.master
        return [(n, self.layout.view(src, i)) for i, n in enumerate(self.names)]

    def _segment_view(self, flat: torch.Tensor, si: int, packed: bool = True) -> torch.Tensor:
        """The elements of segment ``si`` inside ``flat``: a state buffer (moments, reduced gradient; ``packed``) holds only
        the owned segments when the state is sharded, the master weights always keep the full layout."""
        seg = self.layout.segments[si]
        if packed and self._packed_state:
            if not (self.seg_lo <= si < self.seg_hi):
                raise IndexError("segment %d is not owned by this process" % si)
            off = self._pack_off[self.rank][si - self.seg_lo]
            return flat[off:off + seg.length]
        return flat[seg.start:seg.start + seg.length]

    def _full_state(self, flat: torch.Tensor) -> torch.Tensor:
        """A full-layout copy of a state buffer. With sharded state every process contributes the segments it owns
        (collective: every process must call it); otherwise the buffer itself."""
        if not self._packed_state:
            return flat
        lay = self.layout
        full = torch.zeros(lay.total, dtype=flat.dtype, device=flat.device)
        for si in range(self.seg_lo, self.seg_hi):
            seg = lay.segments[si]
            full[seg.start:seg.start + seg.length].copy_(self._segment_view(flat, si))
        for r, (slo, shi) in enumerate(self._owner_ranges):
            for si in range(slo, shi):
                seg = lay.segments[si]
                dist.broadcast(full[seg.start:seg.start + seg.length], src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                               group=self.group)
        return full

    def optimizer_state(self):
        """{name: {"step", "exp_avg", "exp_avg_sq"}} as whole tensors (with sharded state: gathered copies, a collective)."""
        lay = self.layout
        m1, m2 = self._full_state(self.m1), self._full_state(self.m2)
        return {n: {"step": self.opt_step, "exp_avg": lay.view(m1, i), "exp_avg_sq": lay.view(m2, i)} for i, n in enumerate(self.names)}

    def named_grads(self):
        """{name: reduced gradient} as whole tensors (with sharded state: gathered copies, a collective)."""
        red = self._full_state(self.grad_red)
        return {n: self.layout.view(red, i) for i, n in enumerate(self.names)}

    def zero_q_gain_grads(self, step: int, freeze_until_step: int) -> int:
        """Freeze the query gains of the QK norm for the first steps: their reduced gradient is zeroed before the update
        (train/qk_gain_control.py; works on whole or sharded state)."""
        if freeze_until_step <= 0 or step >= freeze_until_step:
            return 0
        n = 0
        for si in (range(self.seg_lo, self.seg_hi) if self.sharded else range(self.n_segs)):
            if self.names[self.layout.segments[si].param].endswith("q_norm.weight"):
                self._segment_view(self.grad_red, si).zero_()
                n += 1
        return n

    def owned_pieces(self) -> list[list[tuple[int, int, dict]]]:
        """Per parameter, the row ranges this process keeps current, each with views of the master weights and the moments
        of those rows: [(row_lo, row_hi, {"weight", "exp_avg", "exp_avg_sq"})]. Adjacent shards are one piece unless the
        state is packed (where each segment has its own place)."""
        lay = self.layout
        out: list[list] = [[] for _ in lay.names]
        if self._packed_state:
            for si in range(self.seg_lo, self.seg_hi):
                seg = lay.segments[si]
                shape = lay.shapes[seg.param]
                row = lay.numels[seg.param] // max(shape[0] if shape else 1, 1)
                lo = (seg.start - lay.offsets[seg.param]) // row
                out[seg.param].append((lo, lo + seg.length // row, {"weight": self._segment_view(self.master, si, packed=False),
                                                                    "exp_avg": self._segment_view(self.m1, si), "exp_avg_sq": self._segment_view(self.m2, si)}))
            for pieces in out:
                pieces.sort(key=lambda t: t[0])
            return out
        for i, rr in enumerate(self.owned_row_ranges()):
            shape = lay.shapes[i]
            row = lay.numels[i] // max(shape[0] if shape else 1, 1)
            for lo, hi in rr:
                a, b = lay.offsets[i] + lo * row, lay.offsets[i] + hi * row
                out[i].append((lo, hi, {"weight": self.master[a:b], "exp_avg": self.m1[a:b], "exp_avg_sq": self.m2[a:b]}))
        return out

    def load_parameter_state(self, i: int, weight: torch.Tensor, exp_avg: torch.Tensor | None, exp_avg_sq: torch.Tensor | None) -> None:
        """Install parameter ``i``'s loaded tensors (whole, on any device): the master weights everywhere, the moments where
        this process keeps them."""
        lay = self.layout
        with torch.no_grad():
            lay.view(self.master, i).copy_(weight)
            if exp_avg is None:
                return
            if not self._packed_state:
                lay.view(self.m1, i).copy_(exp_avg)
                lay.view(self.m2, i).copy_(exp_avg_sq)
                return
            for si in range(self.seg_lo, self.seg_hi):
                seg = lay.segments[si]
                if seg.param != i:
                    continue
                a = seg.start - lay.offsets[i]
                self._segment_view(self.m1, si).copy_(exp_avg.reshape(-1)[a:a + seg.length])
                self._segment_view(self.m2, si).copy_(exp_avg_sq.reshape(-1)[a:a + seg.length])

    def _barrier(self) -> None:
        if self.world > 1:
            if self.is_cuda:
                torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.group)

    def refresh_compute_weights(self) -> None:
        """compute weights <- master (all segments, local only); used at start-up and after a load."""
        K.weight_epoch = (K.weight_epoch or 0) + 1
        if getattr(self, "_pg", None) is not None:  # every process holds the whole master here: nothing left to pull
            for g in self._pg["weights"]:
                g.mark_complete()
        if not self.mixed:
            return
        arr = _ptr_array([self.compute.data_ptr()])
        if self.is_cuda:
            check(self.lib.otb_push_cast(P(self.chunk_start), P(self.chunk_len), I(self.n_chunks), P(self.master), arr, I(1), I(1),
                                         stream_ptr()), "push_cast")
        else:
            check(self.lib.otb_cpu_push_cast(P(self.chunk_start), P(self.chunk_len), I(self.n_chunks), P(self.master), arr, I(1), I(1)),
                  "push_cast")

    # ---------------------------------------------------------------------------- one step
    def forward_backward(self, vslot: int, input_ids: torch.Tensor, labels: torch.Tensor, accum: int, last: bool = False):
        """One micro-batch of hosted virtual rank ``vslot`` (index into ``self.hosted``). ``last``: this is the step's
        final micro-batch on this process, so finished buckets of gradients may enter the reduction during its backward."""
        if self.fold:
            vslot = 0  # every virtual rank is processed in the one work buffer, then folded away
        fresh = self._stale[vslot]
        overlap = last and self._ov is not None and self._begin_overlap(vslot, fresh)
        self._bind_slots(self.grads[vslot], fresh)
        set_tp(self._tp_state)
        if self._tp_state is not None:  # this rank's token rows of the labels
            labels = labels.reshape(-1)[self._tp_state.rows(labels.numel())]
            if self._tp_state.ws is not None:
                # the per-layer peer buffers are reused by every micro-batch: nobody overwrites one while a peer's previous
                # backward pass may still read it (a flag exchange on the stream, no host synchronisation)
                self._tp_state.ws.barrier()
        qat = self.cfg.model.qat
        if qat.enabled and qat.enable_at_step > 0:  # bf16 warm start: a pure function of (step, config)
            set_qat_active(self.model, self._run_step() >= qat.enable_at_step)
        self.model.train()
        self._tick(None)
        z_coeff = self.cfg.model.z_loss.coeff if self.cfg.model.z_loss.enabled else 0.0
        if self.stream_head:
            # vocabulary head and loss in row panels: the [tokens, vocabulary] logits never exist as a whole
            hidden = self.model.forward_hidden(input_ids)
            head = self.model.lm_head
            panel = int(os.environ.get("PRETRAIN_AUDIT_HEAD_CHUNK_ROWS", "2048"))
            ce, z, dh, _ = streaming_head_loss(hidden.detach(), head._cw() if head._cw() is not None else head.weight.detach(), labels,
                                               z_coeff, panel, 1.0 / accum, head._slot())
            self._tick("fwd")
            hidden.backward(dh)
        else:
            self.model.bucket_notify = self._block_done if overlap else None
            try:
                out = self.model(input_ids)
                ce, z = fused_ce_z_loss(out.logits, labels, z_coeff, 1.0 / accum)
                loss = (ce + z) * (1.0 / accum)
                self._tick("fwd")
                loss.backward()
            finally:
                self.model.bucket_notify = None
        self._tick("bwd")
        if fresh:
            unwritten = self._zero_unwritten_slots()
            self._stale[vslot] = False
            if self._ov is not None:
                if overlap and not unwritten <= (self._ov["unwritten"] or set()):
                    raise RuntimeError("parameters %s received no gradient in this micro-batch but did before: their buckets "
                                       "entered the reduction with stale values" % sorted(unwritten - (self._ov["unwritten"] or set())))
                self._ov["unwritten"] = unwritten
        if overlap:
            if self._ov["timeline"] is not None:
                self._bwd_end_event = torch.cuda.Event(enable_timing=True)
                self._bwd_end_event.record()
            for b in range(self.cfg.model.n_layers + 2):  # the embedding, and any bucket no mark reported
                self._launch_bucket(b)
        return ce, z

    def _begin_overlap(self, vslot: int, fresh: bool) -> bool:
        """Prepare the overlapped reduction for this (last) micro-batch; False = reduce after the backward pass as usual."""
        ov = self._ov
        if fresh and ov["unwritten"] is None:
            return False  # which parameters never receive a gradient is learnt from the first backward pass
        for j, stale in enumerate(self._stale):
            if stale and j != vslot:  # a hosted virtual rank without micro-batches contributes zeros
                self.grads[j].zero_()
                self._stale[j] = False
        if fresh:
            for i in ov["unwritten"]:  # nobody will write these: they hold last step's values until zeroed
                self.layout.view(self.grads[vslot], i).zero_()
        ov["epoch"] += 1
        ov["launched"] = set()
        ov["active"] = True
        return True

    def fold_virtual_rank(self, v: int) -> None:
        """Folded-gradient mode: virtual rank ``v`` has run all its micro-batches of this step; add its gradient (the
        work buffer) into its replica's partial. Must be called for v = 0, 1, 2, ... in order."""
        assert self.fold
        S = self.dp_shard
        r, sh = v // S, v % S
        work = self.grads[0]
        if self._stale[0]:
            work.zero_()  # a virtual rank without micro-batches contributes zeros
        if sh == 0:
            part = work.clone()
        else:
            part = self._partials[r]
            part.add_(work)
        if sh == S - 1:
            part.mul_(torch.tensor(1.0, dtype=torch.float32, device=part.device) / torch.tensor(float(S), dtype=torch.float32, device=part.device))
            if self._fold_spill:
                part = self._spill(r, part)
        self._partials[r] = part
        self._stale[0] = True

    def _spill(self, r: int, part: torch.Tensor) -> str:
        """Write a finished replica partial to disk with its blake2b digest beside it; returns the path."""
        import hashlib
        from pathlib import Path

        d = Path(self._fold_spill)
        d.mkdir(parents=True, exist_ok=True)
        path = d / ("replica_%03d.f32" % r)
        raw = part.detach().to("cpu").numpy()
        raw.tofile(path)
        h = hashlib.blake2b(digest_size=32)
        h.update(raw.tobytes())
        Path(str(path) + ".blake2b").write_text(h.hexdigest())
        return str(path)

    def _unspill(self, path: str) -> torch.Tensor:
        import hashlib
        from pathlib import Path

        raw = np.fromfile(path, dtype=np.float32)
        # PRETRAIN_AUDIT_SPILL_VERIFY=0 skips the comparison with the digest written at spill time (on by default: a spill
        # that came back different must stop the audit, not change its answer; reference src/pretrain/cli/audit_replay.py:97-116)
        if os.environ.get("PRETRAIN_AUDIT_SPILL_VERIFY", "1").lower() not in ("0", "false", "no", "off"):
            h = hashlib.blake2b(digest_size=32)
            h.update(raw.tobytes())
            if h.hexdigest() != Path(path + ".blake2b").read_text().strip():
                raise SpillCorruption("%s does not match the digest written beside it" % path)
        return torch.from_numpy(raw).to(self.device)

    def zero_grads(self) -> None:
        """Start a step: every hosted virtual rank's gradient buffer is declared stale. Nothing is written here - the
        first micro-batch of each virtual rank stores its weight gradients (GEMM epilogue without the read), later
        ones accumulate."""
        self._stale = [True] * len(self.grads)

    def reduce_gradients(self) -> float:
        """Steps 2-3: deterministic reduction into ``grad_red`` and the global gradient norm."""
        lay = self.layout
        S, R = self.dp_shard, self.dp_replicate
        per = self.V // self.dp_groups
        self._wait_pending_hash()
        self._tick(None)
        for g, stale in zip(self.grads, self._stale):
            if stale:  # a hosted virtual rank that ran no micro-batch this step contributes zeros, not last step's values
                g.zero_()
        self._stale = [False] * len(self.grads)
        if self.is_cuda:
            wgrad_join()  # weight-gradient GEMMs run on a second stream during the backward pass
        if self._ov is not None and self._ov["active"]:
            # every bucket entered the reduction during the last backward pass; the main stream goes on after the last one
            self._ov["active"] = False
            if self.is_cuda:
                ev = torch.cuda.Event()
                ev.record(self._ov["reduce_stream"])
                torch.cuda.current_stream().wait_event(ev)
            if self.peer:
                self._share_chunk_sos()
            return self._finish_norm()
        if self.tp > 1 and not self.peer:
            # assemble each virtual rank's gradient from the slices its tensor-parallel ranks wrote: at most one rank holds
            # a non-zero bit pattern per element, so the integer sum of the bit patterns is that pattern, exactly
            for g in self.grads:
                dist.all_reduce(g.view(torch.int32), op=dist.ReduceOp.SUM, group=self._tp_state.group)
        if self.nccl_mode and self.world > 1:
            # throughput-only baseline: library all-reduce, order not pinned
            acc = self.grads[0]
            for g in self.grads[1:]:
                acc.add_(g)
            dist.all_reduce(acc, group=self.group)
            self.grad_red.copy_(acc).mul_(1.0 / self.V)
            check(self._chunk_sos_all(), "chunk_sos")
        elif self.collective:
            self._reduce_by_messages(S, R, per)
        elif self.dp_groups > 1 and not self.peer:
            # CPU ranks, and GPU ranks that run tensor-parallel groups: exchange the flat buffers (gloo / NCCL all-gather),
            # then every rank reduces everything identically from its own copies
            gathered = []
            for g in self.grads:
                parts = [torch.empty_like(g) for _ in range(self.world)]
                dist.all_gather(parts, g, group=self.group)
                gathered.append(parts)
            srcs = [gathered[v % per][(v // per) * self.tp].data_ptr() for v in range(self.V)]  # any rank of the owning group
            self._keep = gathered
            if self.is_cuda:
                check(self.lib.otb_grad_reduce(_ptr_array(srcs), I(S), I(R), P(self.chunk_start), P(self.chunk_len), I(self.n_chunks),
                                               P(self.grad_red), P(self.chunk_sos), stream_ptr()), "grad_reduce")
            else:
                check(self.lib.otb_cpu_grad_reduce(_ptr_array(srcs), I(S), I(R), P(self.chunk_start), P(self.chunk_len), I(self.n_chunks),
                                                   P(self.grad_red), P(self.chunk_sos)), "grad_reduce")
            self._keep = None
        else:
            self._stream_barrier()  # every rank's backward is complete before anyone pulls
            srcs = []
            if self.fold:
                # the shard fold and the 1/S scaling are done; what is left is the binary-blocks fold over the R replica partials
                parts = [self._partials[r] for r in range(R)]
                parts = [self._unspill(p) if isinstance(p, str) else p for p in parts]
                self._keep = parts
                srcs, S = [p.data_ptr() for p in parts], 1
                self._partials = {}
            tpn = self.tp if self.peer else 1
            for v in range(self.V if not self.fold else 0):
                r, slot = v // per, v % per
                for t in range(tpn):  # the tensor-parallel ranks of group r hold disjoint slices of virtual rank v's gradient
                    srcs.append(self.buf_grads[slot].ptrs[r * tpn + t] if self.peer else self.grads[slot].data_ptr())
            lo, cnt = self.chunk_lo, self.chunk_hi - self.chunk_lo
            cs, cl = self.chunk_start[lo:], self.chunk_len[lo:]
            sos = self.chunk_sos[lo:]
            sst = self.chunk_state_start[lo:] if self.chunk_state_start is not None else None  # packed reduced gradient
            if self.is_cuda:
                check(self.lib.otb_grad_reduce_ex(_ptr_array(srcs), I(S), I(R), I(tpn), P(cs), P(cl), P(None), I(cnt), P(sst), P(self.grad_red), P(sos),
                                                  stream_ptr()), "grad_reduce")
            else:
                check(self.lib.otb_cpu_grad_reduce_ex(_ptr_array(srcs), I(S), I(R), P(cs), P(cl), P(None), I(cnt), P(sst), P(self.grad_red), P(sos)),
                      "grad_reduce")
            if self.fold:
                self._keep = None
            if self.peer:
                self._share_chunk_sos()
        return self._finish_norm()

    def _finish_norm(self) -> float:
        if self.is_cuda:
            check(self.lib.otb_seg_pair_tree(P(self.chunk_sos), P(self.seg_first), I(self.n_segs), P(self.seg_sos), stream_ptr()), "seg_tree")
        else:
            check(self.lib.otb_cpu_seg_pair_tree(P(self.chunk_sos), P(self.seg_first), I(self.n_segs), P(self.seg_sos)), "seg_tree")
        self._tick("clip")
        seg = self.seg_sos[: self.n_segs].detach().to("cpu").numpy()
        return self._fold_norm(seg)

    # ----------------------------------------------------------------- collective transport (several machines, CPU ranks)
    def _pack(self, flat: torch.Tensor, owner: int) -> torch.Tensor:
        """The segments ``owner`` owns, copied out of a flat buffer into one packed tensor."""
        slo, shi = self._owner_ranges[owner]
        segs, offs = self.layout.segments[slo:shi], self._pack_off[owner]
        if not segs:
            return torch.zeros(self._pack_len[owner], dtype=flat.dtype, device=flat.device)
        # one concatenation (a batched copy) instead of one small copy per segment: the views of the segments with the
        # zero padding that keeps every packed segment on a 64-element boundary
        pieces, end = [], 0
        for sg, off in zip(segs, offs):
            pieces.append(flat[sg.start:sg.start + sg.length])
            end = off + sg.length
            pad = (-sg.length) % 64
            if pad:
                pieces.append(self._zeros(pad, flat))
                end += pad
        if end < self._pack_len[owner]:
            pieces.append(self._zeros(self._pack_len[owner] - end, flat))
        return torch.cat(pieces)

    def _zeros(self, n: int, like: torch.Tensor) -> torch.Tensor:
        cache = self.__dict__.setdefault("_zero_pads", {})
        key = (n, like.dtype)
        if key not in cache:
            cache[key] = torch.zeros(n, dtype=like.dtype, device=like.device)
        return cache[key]

    def _unpack(self, packed: torch.Tensor, owner: int, flat: torch.Tensor) -> None:
        slo, shi = self._owner_ranges[owner]
        segs, offs = self.layout.segments[slo:shi], self._pack_off[owner]
        if segs:  # one batched copy for all segments
            torch._foreach_copy_([flat[sg.start:sg.start + sg.length] for sg in segs], [packed[off:off + sg.length] for sg, off in zip(segs, offs)])

    def _exchange(self, sends: list, recvs: list) -> None:
        """``sends[r]`` goes to process r, ``recvs[p]`` arrives from process p (point-to-point, any backend)."""
        recvs[self.rank].copy_(sends[self.rank])
        ops = []
        for r in range(self.world):
            if r != self.rank:
                peer = dist.get_global_rank(self.group, r) if self.group is not None else r
                ops.append(dist.P2POp(dist.isend, sends[r], peer, group=self.group))
                ops.append(dist.P2POp(dist.irecv, recvs[r], peer, group=self.group))
        for req in dist.batch_isend_irecv(ops) if ops else []:
            req.wait()

    def _reduce_by_messages(self, S: int, R: int, per: int) -> None:
        """Sharded reduction without peer memory: every process sends each owner that owner's segments of every virtual
        rank it hosts; the owner then holds all V copies of its segments and runs the reduction kernel over them - the
        same ascending shard fold and replica tree, on the same values, as the peer-load path."""
        mine = self._pack_len[self.rank]
        got: dict[int, torch.Tensor] = {}
        for j, g in enumerate(self.grads):
            sends = [self._pack(g, r) for r in range(self.world)]
            recvs = [torch.empty(mine, dtype=torch.float32, device=self.device) for _ in range(self.world)]
            self._exchange(sends, recvs)
            for p_, t in enumerate(recvs):
                got[p_ * per + j] = t
        srcs = [got[v].data_ptr() for v in range(self.V)]
        # a packed reduced gradient has exactly the layout of the packed messages
        red = self.grad_red if self._packed_state else torch.empty(mine, dtype=torch.float32, device=self.device)
        lo, cnt = self.chunk_lo, self.chunk_hi - self.chunk_lo
        cl, sos = self.chunk_len[lo:], self.chunk_sos[lo:]
        if self.is_cuda:
            check(self.lib.otb_grad_reduce(_ptr_array(srcs), I(S), I(R), P(self._packed_chunk_start), P(cl), I(cnt), P(red), P(sos), stream_ptr()),
                  "grad_reduce")
        else:
            check(self.lib.otb_cpu_grad_reduce(_ptr_array(srcs), I(S), I(R), P(self._packed_chunk_start), P(cl), I(cnt), P(red), P(sos)), "grad_reduce")
        if not self._packed_state:
            self._unpack(red, self.rank, self.grad_red)
        self._share_chunk_sos()

    def _share_chunk_sos(self) -> None:
        """Every process learns the squared-norm partials of the chunks the others own."""
        lay = self.layout
        parts = [torch.empty_like(self.chunk_sos) for _ in range(self.world)]
        dist.all_gather(parts, self.chunk_sos, group=self.group)
        for r, (slo, shi) in enumerate(lay.owner_ranges(self.world)):
            c0, c1 = int(lay.seg_first[slo]), int(lay.seg_first[shi])
            if r != self.rank and c1 > c0:
                self.chunk_sos[c0:c1].copy_(parts[r][c0:c1])

    def _share_updated_weights(self) -> None:
        """After the update of the owned segments: every process receives the others' new compute weights."""
        width = max(self._pack_len)
        mine = torch.zeros(width, dtype=self.compute.dtype, device=self.device)
        mine[: self._pack_len[self.rank]].copy_(self._pack(self.compute, self.rank))
        carrier = mine.view(torch.uint8)  # byte transport (gloo has no bf16 type)
        parts = [torch.empty_like(carrier) for _ in range(self.world)]
        dist.all_gather(parts, carrier, group=self.group)
        for r in range(self.world):
            if r != self.rank:
                self._unpack(parts[r].view(self.compute.dtype), r, self.compute)

    def _chunk_sos_all(self) -> int:
        if self.is_cuda:
            return self.lib.otb_chunk_sos(P(self.grad_red), P(self.chunk_start), P(self.chunk_len), I(self.n_chunks), P(self.chunk_sos), stream_ptr())
        return self.lib.otb_cpu_chunk_sos(P(self.grad_red), P(self.chunk_start), P(self.chunk_len), I(self.n_chunks), P(self.chunk_sos))

    def _fold_norm(self, seg_sos: np.ndarray) -> float:
        """per-tensor sum over shards ascending, then over tensors ascending, all in fp32; then sqrt.
        (grad_norm_algo = deterministic_per_tensor_sos_v1)"""
        per_tensor = np.zeros(len(self.names), dtype=np.float32)
        seen = np.zeros(len(self.names), dtype=bool)
        order = sorted(range(self.n_segs), key=lambda i: (self.layout.segments[i].param, self.layout.segments[i].shard))
        for i in order:
            pi = self.layout.segments[i].param
            per_tensor[pi] = seg_sos[i] if not seen[pi] else np.float32(per_tensor[pi] + seg_sos[i])
            seen[pi] = True
        self.per_tensor_sos = per_tensor
        total = np.float32(0.0)
        for v in per_tensor:
            total = np.float32(total + v)
        return float(np.sqrt(total, dtype=np.float32))

    @staticmethod
    def clip_coefficient(grad_norm: float, max_norm: float) -> float:
        if max_norm <= 0:
            return 1.0
        h = np.float32(max_norm) / np.float32(np.float32(grad_norm) + np.float32(1e-6))
        return float(min(h, np.float32(1.0)))

    def _run_step(self) -> int:
        """Index of the step being computed: the run's step counter when the caller maintains `global_step` (it keeps
        counting through skipped steps and through a resume that resets the optimizer), else the optimizer's own."""
        return self.opt_step if self.global_step is None else int(self.global_step)

    def optimizer_step(self, lr: float, clip: float) -> None:
        """Step 4 on the owned segments; pushes the new weights to every rank."""
        self._wait_pending_hash()
        self._tick(None)
        self.opt_step += 1
        for g in self.param_groups:
            g["lr"] = float(lr)
        o = self.cfg.optim
        hyper = (ctypes.c_float * 10)()
        cpu_lib().otb_cpu_adamw_hyper(ctypes.c_double(lr), ctypes.c_double(o.betas[0]), ctypes.c_double(o.betas[1]), ctypes.c_double(o.eps),
                                      ctypes.c_double(o.weight_decay), ctypes.c_long(self.opt_step), F(clip), hyper)
        lo, cnt = self.chunk_lo, self.chunk_hi - self.chunk_lo
        cs, cl, cg = self.chunk_start[lo:], self.chunk_len[lo:], self.chunk_group[lo:]
        if self.muon_params:
            cs, cl, cg, cnt = self._aux_chunks
            self._muon_step(float(lr), float(clip))
        dst_buf = self.buf_compute
        dsts = dst_buf.ptrs if self.peer else [self.compute.data_ptr()]
        sst = None
        if self.chunk_state_start is not None and not self.muon_params:
            sst = self.chunk_state_start[lo:]  # gradient and moments sit in the packed buffers of the owned segments
        launches = [(cs, sst, cl, cg, cnt, dsts)]
        if self._pg is not None:
            # gather mode: the rows of the projection weights stay on their owner (the consuming GEMM pulls them), the
            # rest (embedding, gains) goes to every GPU as before
            own = [self.compute.data_ptr()]
            launches = [(t[0], t[3], t[1], t[2], t[4], d) for t, d in ((self._pg["tables"]["pull"], own), (self._pg["tables"]["push"], dsts))]
        for cs_, sst_, cl_, cg_, cnt_, dsts_ in launches:
            if self.is_cuda:
                check(self.lib.otb_adamw_push_ex(hyper, P(cs_), P(sst_), P(cl_), P(cg_), I(cnt_), P(self.master), P(self.grad_red), P(self.m1), P(self.m2),
                                                 _ptr_array(dsts_), I(len(dsts_)), I(self.mixed), stream_ptr()), "adamw_push")
            else:
                check(self.lib.otb_cpu_adamw_push_ex(hyper, P(cs_), P(sst_), P(cl_), P(cg_), I(cnt_), P(self.master), P(self.grad_red), P(self.m1), P(self.m2),
                                                     _ptr_array(dsts_), I(len(dsts_)), I(self.mixed)), "adamw_push")
        if self._pg is not None:
            self._pg["epoch"] += 1
            for g in self._pg["weights"]:
                g.epoch = self._pg["epoch"]
        if self.collective:
            self._share_updated_weights()
        self._tick("opt")
        self._stream_barrier()  # peers' stores into this rank's weights are complete before the next forward
        K.weight_epoch = (K.weight_epoch or 0) + 1
        self._refresh_scales_if_due(self.opt_step if self.global_step is None else int(self.global_step) + 1)

    def _refresh_scales_if_due(self, steps_done: int) -> None:
        """After the update (or the skipped update), before the state hash: every rank derives the same LSQ step sizes
        from its (identical) compute weights (reference src/pretrain/train/loop.py:1069-1084; it runs on skipped steps too)."""
        refresh = self.cfg.model.qat.scale_refresh_every_n_steps
        if self.cfg.model.qat.enabled and refresh > 0 and steps_done % refresh == 0:
            refresh_lsq_weight_scales(self.model)
            K.weight_epoch = (K.weight_epoch or 0) + 1

    def _muon_step(self, lr: float, clip: float) -> None:
        """Muon on the hidden matrices: momentum (kept in the first-moment buffer; the second stays zero), Nesterov
        look-ahead, five Newton-Schulz iterations in bf16, decoupled weight decay; then the compute copies follow."""
        from ..optim.muon import newton_schulz5

        lay, o = self.layout, self.cfg.optim
        mom = float(o.betas[1])
        with torch.no_grad():
            for i in self.muon_params:
                p, g, buf = lay.view(self.master, i), lay.view(self.grad_red, i), lay.view(self.m1, i)
                if clip != 1.0:
                    g.mul_(clip)
                buf.mul_(mom).add_(g)
                upd = newton_schulz5(g.add(buf, alpha=mom))
                if o.weight_decay:
                    p.mul_(1.0 - lr * o.weight_decay)
                p.add_(upd, alpha=-lr * max(1.0, p.shape[0] / p.shape[1]) ** 0.5)
                if self.mixed:
                    lay.view(self.compute, i).copy_(p)

    def skip_step(self) -> None:
        self._stream_barrier()  # nobody overwrites a gradient buffer that a peer may still be reading
        if self.global_step is not None:
            self._refresh_scales_if_due(int(self.global_step) + 1)

    # --------------------------------------------------------------------------------- hash
    def _hash_fields(self, include_grads: bool):
        return [("weight", self.master), ("exp_avg", self.m1), ("exp_avg_sq", self.m2)] + ([("grad", self.grad_red)] if include_grads else [])

    def _wait_pending_hash(self) -> None:
        """Kernels that overwrite hashed state wait (on the device) for a state hash still running on the side stream."""
        ev = getattr(self, "_hash_done", None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self._hash_done = None

    def begin_state_hash(self, include_grads: bool = True, tensor_digest: str | None = None) -> dict:
        """Start the v3 hash of the CURRENT state and return a handle for ``finish_state_hash``. With tree digests on a
        GPU the per-segment digests are computed on a low-priority side stream, so the next step's forward and backward
        (which touch neither the master weights, the moments nor the reduced gradient) run on top of them; the kernels
        that do overwrite that state (gradient reduction, optimizer step) wait for the digests first."""
        td = tensor_digest or self.cfg.train.state_hash.tensor_digest
        lay = self.layout
        if self.sharded and td != "tree":
            raise ValueError("sharded multi-GPU hashing needs train.state_hash.tensor_digest=tree")
        handle = {"td": td, "include_grads": include_grads, "opt_step": self.opt_step, "keys": None, "plan": None, "digests": None}
        if td != "tree":
            return handle
        fields = self._hash_fields(include_grads)
        keys, views = [], []
        for si in range(self.seg_lo, self.seg_hi) if self.sharded else range(self.n_segs):
            seg = lay.segments[si]
            for tag, flat in fields:
                keys.append((seg.param, seg.shard, tag))
                views.append(self._segment_view(flat, si, packed=tag != "weight"))
        handle["keys"] = keys
        if self.is_cuda and views:
            plans = self.__dict__.setdefault("_hash_plans", {})
            plan = plans.get(include_grads)
            if plan is None:
                plan = plans[include_grads] = SH.TreeDigestPlan(views)
                lo, _hi = torch.cuda.Stream.priority_range()
                self._hash_stream = getattr(self, "_hash_stream", None) or torch.cuda.Stream(device=self.device, priority=lo)
            ready = torch.cuda.Event()
            ready.record()
            self._hash_stream.wait_event(ready)
            plan.launch(self._hash_stream)
            done = torch.cuda.Event()
            done.record(self._hash_stream)
            self._hash_done = done
            handle["plan"], handle["done"] = plan, done
        else:
            handle["digests"] = SH.tree_digest_batch(views)
        return handle

    def finish_state_hash(self, handle: dict, prev, batch_digest: bytes | None) -> str:
        """Complete a hash started by ``begin_state_hash``: wait for the digests, gather them from the other processes
        when ownership is sharded, and fold everything into the v3 byte stream on the host."""
        td, include_grads = handle["td"], handle["include_grads"]
        lay = self.layout
        seg_digests = {}
        if td == "tree":
            if handle["plan"] is not None:
                handle["done"].synchronize()
                digs = handle["plan"].digests()
            else:
                digs = handle["digests"]
            seg_digests = dict(zip(handle["keys"], digs))
            if self.sharded:
                # every process knows which (parameter, shard, field) digests every other one owns, so only the 32-byte
                # values travel: one all-gather of a fixed-size byte tensor
                cache = self.__dict__.setdefault("_hash_keys_by_rank", {})
                keys_by_rank = cache.get(include_grads)
                if keys_by_rank is None:
                    fields = [tag for tag, _ in self._hash_fields(include_grads)]
                    keys_by_rank = cache[include_grads] = [
                        [(lay.segments[si].param, lay.segments[si].shard, tag) for si in range(slo, shi) for tag in fields]
                        for slo, shi in lay.owner_ranges(self.world)]
                width = 32 * max(max(len(k) for k in keys_by_rank), 1)
                mine = torch.zeros(width, dtype=torch.uint8)
                raw = b"".join(digs)
                mine[: len(raw)] = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
                if self._host_gloo:  # the digests are host bytes already: no reason to touch the device or its streams
                    parts = [torch.empty_like(mine) for _ in range(self.world)]
                    dist.all_gather(parts, mine, group=self.host_group)
                else:
                    mine = mine.to(self.device)
                    parts = [torch.empty_like(mine) for _ in range(self.world)]
                    dist.all_gather(parts, mine, group=self.group)
                allraw = torch.stack(parts).cpu().numpy().tobytes()
                seg_digests = {}
                for r, keys in enumerate(keys_by_rank):
                    base = r * width
                    for j, k in enumerate(keys):
                        seg_digests[k] = allraw[base + 32 * j: base + 32 * j + 32]
        order = sorted(range(len(self.names)), key=lambda i: self.names[i])
        step_bytes = b"optim_step\0" + int(handle["opt_step"]).to_bytes(8, "little", signed=True)
        empty = SH.tree_digest_bytes(b"") if td == "tree" else None
        locals_ = []
        for s in range(self.dp_shard):
            h = SH._new()
            for pi in order:
                shape = lay.shapes[pi] if lay.shapes[pi] else (1,)
                lo, hi = SH.shard_rows(shape[0], self.dp_shard, s)
                sshape = (hi - lo,) + tuple(shape[1:])
                h.update(self.names[pi].encode() + b"\0")
                head = b"\0torch.float32\0" + str(sshape).encode() + b"\0"

                def feed(tag, key, flat):
                    if td == "tree":
                        h.update(tag + head + b"tree\0" + (seg_digests[(pi, s, key)] if hi > lo else empty))
                    else:
                        h.update(tag + head)
                        row = lay.numels[pi] // max(shape[0], 1)
                        st = lay.offsets[pi] + lo * row
                        SH.feed_raw(h, flat[st:st + (hi - lo) * row])

                feed(b"weight", "weight", self.master)
                h.update(step_bytes)
                feed(b"optim_exp_avg", "exp_avg", self.m1)
                feed(b"optim_exp_avg_sq", "exp_avg_sq", self.m2)
                if include_grads:
                    feed(b"grad", "grad", self.grad_red)
            locals_.append(h.digest())
        shard_state = SH.combine_shard_state(locals_, self.V)
        return SH.finalize_state_hash(shard_state, self.param_groups, prev, batch_digest)

    def sharded_state_hash(self, prev, batch_digest: bytes | None, include_grads: bool = True, tensor_digest: str | None = None) -> str:
        """v3 hash of the current state. With peer-sharded ownership each process digests the segments it
        owns (tree digests, on the device) and the 32-byte results are gathered."""
        return self.finish_state_hash(self.begin_state_hash(include_grads, tensor_digest), prev, batch_digest)

    def full_state_hash(self, prev=None, batch_digest=None, include_grads: bool = False) -> str:
        """v2 hash over full tensors (init hash). Only valid where this process holds every segment."""
        grads = self.named_grads() if include_grads else None
        return SH.compute_state_hash(self.named_master(), self.optimizer_state(), self.param_groups, prev=prev,
                                     include_grads=include_grads, grads=grads, batch_digest=batch_digest)

    def owned_row_ranges(self) -> list[list[tuple[int, int]]]:
        """Per parameter, the row ranges [lo, hi) whose master weights and moments THIS process keeps current (adjacent
        virtual shards merged). With sharded ownership: the rows of its segments; otherwise every process holds the whole
        state and rank 0 stands for all of them."""
        lay = self.layout
        out: list[list[tuple[int, int]]] = [[] for _ in lay.names]
        if self.sharded:
            segs = lay.segments[self.seg_lo:self.seg_hi]
        else:
            segs = lay.segments if self.rank == 0 else []
        for sg in sorted(segs, key=lambda g: (g.param, g.shard)):
            shape = lay.shapes[sg.param]
            dim0 = shape[0] if shape else 1
            row = lay.numels[sg.param] // max(dim0, 1)
            lo = (sg.start - lay.offsets[sg.param]) // row
            hi = lo + sg.length // row
            rr = out[sg.param]
            if rr and rr[-1][1] == lo:
                rr[-1] = (rr[-1][0], hi)
            else:
                rr.append((lo, hi))
        return out

    def gather_full_state(self) -> None:
        """Make master / moments / reduced gradient complete on every rank (checkpoint, init hash)."""
        if not self.sharded:
            return
        self._wait_pending_hash()
        lay = self.layout
        ranges = lay.owner_ranges(self.world)
        for flat in ((self.master,) if self._packed_state else (self.master, self.m1, self.m2, self.grad_red)):
            for r, (slo, shi) in enumerate(ranges):
                for si in range(slo, shi):
                    seg = lay.segments[si]
                    dist.broadcast(flat[seg.start:seg.start + seg.length], src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                                   group=self.group)

    def close(self) -> None:
        if self._tp_state is not None and self._tp_state.ws is not None:
            self._tp_state.ws.close()
            self._tp_state.ws = None
        extra = [self._ov[k] for k in ("flags", "bar") if self._ov is not None and k in self._ov]
        for b in [self.buf_master, self.buf_compute] + self.buf_grads + extra:
            b.close()
        self._off_files.clear()
        for tmp in self._off_tmp:
            try:
                tmp.cleanup()
            except OSError:
                pass
        self._off_tmp = []
