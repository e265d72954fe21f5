"""torch.autograd bindings of the native kernels.

Weight gradients do not travel through ``.grad``: a parameter may carry a *gradient slot*
(``GradSlot``), an fp32 view into the flat gradient buffer of the virtual rank currently being
processed, and the weight-gradient GEMM accumulates straight into it (fp32, beta = 1 epilogue).
Without a slot the functions return ordinary gradients, so the same modules serve evaluation,
tests and the audit replay.
"""
from __future__ import annotations

import math
import os

import torch
from torch.autograd import Function

from . import functional as K


class GradSlot:
    """fp32 accumulation target of one parameter (a view into a flat gradient buffer).

    ``fresh`` means the buffer's current contents are stale (first micro-batch of a virtual rank in this step): the
    first writer STORES its result instead of accumulating, which spares the step a 4-byte-per-parameter memset and the
    read half of the accumulate, and sets ``written``. Whoever owns the slots zeroes those still unwritten after the
    backward pass (parameters that received no gradient)."""

    __slots__ = ("buf", "fresh", "written", "gather")

    def __init__(self, buf: torch.Tensor | None = None):
        self.buf = buf
        self.fresh = False
        self.written = False
        # parallel/param_gather.py::GatheredWeight when the weight's rows are pulled from their owners by the first
        # forward GEMM after an update (``run.param_sharding: gather``), else None
        self.gather = None

    def take(self) -> bool:
        """True if the caller must overwrite (store); later callers accumulate."""
        first = self.fresh and not self.written
        self.written = True
        return first

    def zero_if_first(self) -> None:
        """For writers that can only accumulate: clear a stale buffer before the first accumulation."""
        if self.take():
            self.buf.zero_()


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


# Weight-gradient GEMMs that accumulate into a gradient slot are not on the critical path of the backward pass (only the
# data gradient feeds the next layer), and their grids end in a partly filled last wave (few output tiles, very long K).
# On a GPU they are therefore issued on a second stream: when the last wave of one GEMM leaves SMs idle, CTAs of the
# kernel queued on the other stream take them. Each kernel still owns its output elements and its summation order, so
# the bits do not change. ``wgrad_join`` makes the current stream wait for everything issued there (the engine calls it
# before the gradient reduction). Off by default (OTB_WGRAD_STREAM=1 turns it on): under the 1 kW power cap the step is
# energy-bound, so filling idle SMs lowers the clock instead of the step time (measured: 1343 vs 1346 ms).
_wgrad_streams: dict = {}
_wgrad_on = os.environ.get("OTB_WGRAD_STREAM", "0") == "1"


def _wgrad_stream(device: torch.device) -> "torch.cuda.Stream":
    st = _wgrad_streams.get(device)
    if st is None:
        st = _wgrad_streams[device] = torch.cuda.Stream(device=device)
    return st


def wgrad_join() -> None:
    """The current stream waits for every weight-gradient GEMM issued on the side stream of its device."""
    if not torch.cuda.is_available():
        return
    st = _wgrad_streams.get(torch.device("cuda", torch.cuda.current_device()))
    if st is not None:
        ev = torch.cuda.Event()
        ev.record(st)
        torch.cuda.current_stream().wait_event(ev)


class BucketMarkFn(Function):
    """Identity in the forward pass. In the backward pass it tells `notify(bucket)` that the gradient with respect to
    this point of the residual stream is complete, i.e. that every layer AFTER this point has run its backward and
    written its weight gradients; the engine starts that bucket's gradient reduction under the rest of the backward."""

    @staticmethod
    def forward(ctx, x, notify, bucket):
        ctx.notify, ctx.bucket = notify, bucket
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        ctx.notify(ctx.bucket)
        return dy, None, None


def bucket_mark(x, notify, bucket):
    return BucketMarkFn.apply(x, notify, bucket)


class LinearFn(Function):
    """y = x W^T (+ residual). ``master`` is the fp32 parameter autograd knows about, ``w`` the
    compute-dtype weight actually multiplied (the same tensor in fp32 runs)."""

    @staticmethod
    def forward(ctx, x, master, w, slot, residual):
        x2 = _flat2d(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pull = slot.gather if slot is not None else None
        if pull is not None and pull.pending():
            # first use of this weight since its owners updated it: the GEMM gathers the missing rows itself
            y = pull.gemm(x2, _flat2d(residual) if residual is not None else None)
        elif residual is not None:
            y = K.gemm(x2, w, epi=K.EPI_RESIDUAL, residual=_flat2d(residual))
        else:
            y = K.gemm(x2, w)
        ctx.save_for_backward(x2, w)
        ctx.slot = slot
        ctx.has_res = residual is not None
        ctx.in_shape = x.shape
        ctx.master_dtype = master.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _flat2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_mn=True).view(ctx.in_shape)
        gm = None
        if ctx.slot is not None and ctx.slot.buf is not None:
            if dy2.is_cuda and _wgrad_on:
                side = _wgrad_stream(dy2.device)
                ready = torch.cuda.Event()
                ready.record()
                side.wait_event(ready)  # dy exists; earlier accumulations into this slot were issued on `side` too
                epi = K.EPI_STORE_F32 if ctx.slot.take() else K.EPI_ACC_F32
                with torch.cuda.stream(side):
                    K.gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.slot.buf, epi=epi)
                dy2.record_stream(side)  # the allocator must not hand these blocks out again before the GEMM has read them
                x2.record_stream(side)
            else:
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.slot.buf, epi=K.EPI_STORE_F32 if ctx.slot.take() else K.EPI_ACC_F32)
        elif ctx.needs_input_grad[1]:
            gm = K.gemm(dy2, x2, a_mn=True, b_mn=True, epi=K.EPI_STORE_F32).to(ctx.master_dtype)
        return dx, gm, None, None, (dy if ctx.has_res else None)


def linear(x, master, w=None, slot=None, residual=None):
    return LinearFn.apply(x, master, master if w is None else w, slot, residual)


# ----------------------------------------------------------------------------- tensor parallelism
# A tensor-parallel group of P processes works on ONE micro-batch together. The residual stream is sharded by token
# rows (rank t holds rows [t M/P, (t+1) M/P) of the flattened [B*T] tokens), the projections are split the Megatron way
# (column-parallel: QKV, gate/up; row-parallel: attention output, FFN down), and the vocabulary head stays token-sharded.
# Every weight is still held in full by every process (the engine replicates the compute weights), so "parallel" here
# means who multiplies which slice. The rule that keeps the bits of the unsplit model: whenever a reduction index
# (features of a column-parallel layer in its data gradient, the inner dimension of a row-parallel layer, tokens in a
# weight gradient) would be split over ranks, the operand is first brought together in the canonical order of the
# unsplit layout and the owner of the output rows runs ONE GEMM over the whole index, ascending. Gradients of a weight
# slice are written by the rank that owns the slice; everything else in that rank's gradient buffer stays zero, and the
# engine assembles a virtual rank's gradient as the element-wise integer sum over the group (at most one non-zero bit
# pattern per element, so the assembly is exact). The collectives are torch.distributed all-gathers on the group (gloo
# on CPU ranks, NCCL on GPUs); the fused peer-memory kernels of parallel/tensor_parallel.py implement the same two
# patterns for the column- and row-parallel forward on GPUs.
class TpState:
    def __init__(self, group, rank: int, size: int):
        self.group, self.rank, self.size = group, rank, size
        self.batch_shape = None  # (B, T) of the micro-batch being processed
        # peer-memory workspace (parallel.tensor_parallel.TpWorkspace) when the fused all-gather -> GEMM and chained
        # GEMM -> ordered-reduction kernels carry the group's traffic instead of library all-gathers; None otherwise
        self.ws = None

    def fused(self, x: torch.Tensor, M: int) -> bool:
        """Whether the peer-memory kernels take this call: bf16 activations on a GPU, whole 128-row blocks per rank."""
        on_device = x.is_cuda or getattr(self.ws, "any_device", False)  # (a host stand-in of the workspace, for tests)
        return self.ws is not None and on_device and x.dtype == torch.bfloat16 and M % (self.size * 128) == 0

    def rows(self, M: int) -> slice:
        assert M % self.size == 0, "token count %d does not split over %d tensor-parallel ranks" % (M, self.size)
        per = M // self.size
        return slice(self.rank * per, (self.rank + 1) * per)

    def split(self, n: int, rank: int | None = None) -> tuple[int, int]:
        assert n % self.size == 0, "%d does not split over %d tensor-parallel ranks" % (n, self.size)
        per = n // self.size
        r = self.rank if rank is None else rank
        return r * per, (r + 1) * per


_TP: TpState | None = None


def set_tp(state: TpState | None) -> None:
    global _TP
    _TP = state if (state is not None and state.size > 1) else None


def tp() -> TpState | None:
    return _TP


def _all_gather(x: torch.Tensor) -> list[torch.Tensor]:
    import torch.distributed as dist

    x = x.contiguous()
    carrier = x.view(torch.uint8) if x.dtype == torch.bfloat16 else x  # byte transport; gloo has no bf16 type
    parts = [torch.empty_like(carrier) for _ in range(_TP.size)]
    dist.all_gather(parts, carrier, group=_TP.group)
    return [p.view(x.dtype) for p in parts] if carrier is not x else parts


def tp_gather_rows(x_shard: torch.Tensor) -> torch.Tensor:
    """[m, ...] per rank -> [m * P, ...], rank order (one collective straight into the result, no concatenation copy)."""
    import torch.distributed as dist

    x = x_shard.contiguous()
    out = torch.empty((x.shape[0] * _TP.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.dtype == torch.bfloat16:  # byte transport; gloo has no bf16 type
        dist.all_gather_into_tensor(out.view(torch.uint8), x.view(torch.uint8), group=_TP.group)
    else:
        dist.all_gather_into_tensor(out, x, group=_TP.group)
    return out


def tp_gather_cols(y_t: torch.Tensor, slices_by_rank, n_total: int) -> torch.Tensor:
    """[M, n_t] per rank -> [M, n_total] with rank r's columns placed at ``slices_by_rank[r]`` (a list of (start, stop)
    in the unsplit layout, consumed left to right)."""
    parts = _all_gather(y_t)
    out = torch.empty((y_t.shape[0], n_total), dtype=y_t.dtype, device=y_t.device)
    for r, sl in enumerate(slices_by_rank):
        off = 0
        for a, b in sl:
            out[:, a:b] = parts[r][:, off:off + (b - a)]
            off += b - a
    return out


def _tp_slot(slot) -> "GradSlot":
    if slot is None or slot.buf is None:
        raise NotImplementedError("tensor-parallel layers accumulate into gradient slots (training engine only)")
    if slot.take():
        slot.buf.zero_()  # the other ranks' slices of this parameter must read zero in this rank's buffer
    return slot


class TpColumnLinearFn(Function):
    """Column-parallel y_t = gather_rows(x) W_t^T: rank t owns the output features ``slices_by_rank[t]`` of W [N, K]."""

    @staticmethod
    def forward(ctx, x_shard, master, w, slot, slices_by_rank):
        st = _TP
        mine = slices_by_rank[st.rank]
        w_t = w[mine[0][0]:mine[0][1]] if len(mine) == 1 else torch.cat([w[a:b] for a, b in mine], 0)
        x2 = _flat2d(x_shard)
        if st.fused(x2, x2.shape[0] * st.size):
            # one kernel: this rank's rows go to the peers' buffers while the tensor-core CTAs start on the local rows;
            # the gathered activation stays in the (per-layer) peer buffer for the weight gradient
            y, x_full = st.ws.ag_gemm(("col", master.data_ptr()), x2.contiguous(), w_t.contiguous())
        else:
            x_full = tp_gather_rows(x2)
            y = K.gemm(x_full, w_t.contiguous())
        ctx.save_for_backward(x_full, w)
        ctx.slot, ctx.slices = slot, slices_by_rank
        return y

    @staticmethod
    def backward(ctx, dy_t):
        x_full, w = ctx.saved_tensors
        st = _TP
        dy_t = dy_t.contiguous()
        slot = _tp_slot(ctx.slot)
        off = 0
        for a, b in ctx.slices[st.rank]:  # weight gradient of the owned rows: every token, ascending
            K.gemm(dy_t[:, off:off + (b - a)], x_full, a_mn=True, b_mn=True, out=slot.buf[a:b], epi=K.EPI_ACC_F32)
            off += b - a
        # data gradient: the reduction runs over ALL output features in the unsplit order, for this rank's token rows
        dy_full = tp_gather_cols(dy_t, ctx.slices, w.shape[0])
        dx = K.gemm(dy_full[st.rows(dy_full.shape[0])].contiguous(), w, b_mn=True)
        return dx, None, None, None, None


class TpRowLinearFn(Function):
    """Row-parallel y = a W^T (+ residual) with the inner dimension split: rank t holds columns ``cols_by_rank[t]`` of
    ``a``; the result comes back sharded by token rows."""

    @staticmethod
    def forward(ctx, a_t, master, w, slot, residual_shard, cols_by_rank):
        st = _TP
        a_t = _flat2d(a_t).contiguous()
        ascending = all(cols_by_rank[r][1] == cols_by_rank[r + 1][0] for r in range(st.size - 1))
        if st.fused(a_t, a_t.shape[0]) and ascending:
            # the fp32 accumulator tile travels rank 0 -> ... -> P-1, each rank continuing the ascending-k accumulation
            # in tensor memory; the last rank stores every tile at the owner of its token rows
            a0, b0 = cols_by_rank[st.rank]
            res = _flat2d(residual_shard).contiguous() if residual_shard is not None else None
            y = st.ws.chain_gemm(("row", master.data_ptr()), a_t, w[:, a0:b0].contiguous(), residual_shard=res)
        else:
            a_full = tp_gather_cols(a_t, [[c] for c in cols_by_rank], w.shape[1])
            mine = a_full[st.rows(a_full.shape[0])].contiguous()
            if residual_shard is not None:
                y = K.gemm(mine, w, epi=K.EPI_RESIDUAL, residual=_flat2d(residual_shard))
            else:
                y = K.gemm(mine, w)
        ctx.master_key = master.data_ptr()
        ctx.save_for_backward(a_t, w)
        ctx.slot, ctx.cols, ctx.has_res = slot, cols_by_rank, residual_shard is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        a_t, w = ctx.saved_tensors
        st = _TP
        a, b = ctx.cols[st.rank]
        dy_shard = dy_shard.contiguous()
        if st.fused(dy_shard, dy_shard.shape[0] * st.size):
            da_t, dy_full = st.ws.ag_gemm(("row_bwd", ctx.master_key), dy_shard, w[:, a:b].contiguous(), b_mn=True)
        else:
            dy_full = tp_gather_rows(dy_shard)
            da_t = K.gemm(dy_full, w[:, a:b], b_mn=True)
        slot = _tp_slot(ctx.slot)
        K.gemm(dy_full, a_t, a_mn=True, b_mn=True, out=slot.buf[:, a:b], epi=K.EPI_ACC_F32)
        return da_t, None, None, None, (dy_shard if ctx.has_res else None), None


class TpTokenLinearFn(Function):
    """Token-sharded linear layer with the full weight (the vocabulary head): forward and data gradient are local to
    the rank's token rows; the weight gradient needs every token, so rank t forms the rows ``split(N, t)`` of dW from the
    gathered dy columns and the gathered input."""

    @staticmethod
    def forward(ctx, x_shard, master, w, slot):
        x2 = _flat2d(x_shard).contiguous()
        ctx.save_for_backward(x2, w)
        ctx.slot = slot
        return K.gemm(x2, w)

    @staticmethod
    def backward(ctx, dy_shard):
        x2, w = ctx.saved_tensors
        st = _TP
        dy_shard = dy_shard.contiguous()
        dx = K.gemm(dy_shard, w, b_mn=True)
        a, b = st.split(w.shape[0])
        dy_cols = None
        for r in range(st.size):  # a transpose of the sharding: rank r collects columns split(N, r) of every rank's rows
            ra, rb = st.split(w.shape[0], r)
            got = tp_gather_rows(dy_shard[:, ra:rb].contiguous())
            if r == st.rank:
                dy_cols = got
        x_full = tp_gather_rows(x2)
        slot = _tp_slot(ctx.slot)
        K.gemm(dy_cols, x_full, a_mn=True, b_mn=True, out=slot.buf[a:b], epi=K.EPI_ACC_F32)
        return dx, None, None, None


def tp_column_linear(x_shard, master, w, slot, slices_by_rank):
    return TpColumnLinearFn.apply(x_shard, master, w, slot, slices_by_rank)


def tp_row_linear(a_t, master, w, slot, residual_shard, cols_by_rank):
    return TpRowLinearFn.apply(a_t, master, w, slot, residual_shard, cols_by_rank)


def tp_token_linear(x_shard, master, w, slot):
    return TpTokenLinearFn.apply(x_shard, master, w, slot)


class RMSNormFn(Function):
    @staticmethod
    def forward(ctx, x, master, w, slot, eps, tp_heads=0):
        x2 = _flat2d(x).contiguous()
        y, rstd = K.rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, rstd, w if w is not None else x2.new_empty(0))
        ctx.has_w = w is not None
        ctx.slot = slot
        ctx.tp_heads = int(tp_heads)
        ctx.shape = x.shape
        ctx.master_dtype = master.dtype if master is not None else None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd, w = ctx.saved_tensors
        w = w if ctx.has_w else None
        dy2 = _flat2d(dy).contiguous()
        need_dg = ctx.has_w and ((ctx.slot is not None and ctx.slot.buf is not None) or ctx.needs_input_grad[1])
        dx, dg = K.rmsnorm_bwd(dy2, x2, w, rstd, need_dg)
        gm = None
        if need_dg and _TP is not None and ctx.tp_heads:
            # rows are (token, head) pairs and the HEADS are split over the group, so a rank's rows interleave with the
            # others' in the unsplit order and its 8-row slabs are not slabs of the unsplit tree: the operands are
            # gathered, put back into (token, all heads) order, and rank 0 runs the gain gradient over the whole of them
            h, P_ = ctx.tp_heads, _TP.size

            def canon(t):
                parts = torch.stack([p.reshape(-1, h, *t.shape[1:]) for p in _all_gather(t)], 1)  # [tokens, P, h, ...]
                return parts.reshape(-1, *t.shape[1:]).contiguous()

            dy_f, x_f, rstd_f = canon(dy2), canon(x2), canon(rstd)
            if _TP.rank == 0:
                _, dg = K.rmsnorm_bwd(dy_f, x_f, w, rstd_f, True)
            else:
                need_dg = False
        elif need_dg and _TP is not None:
            # each rank's dg is the root of the slab pair tree over its own token rows (a sub-tree of the unsplit tree when
            # the rank holds a power-of-two number of slabs); the roots are combined in rank order by the same tree, and
            # rank 0 alone adds the result to its gradient buffer
            n_slabs = (x2.shape[0] + K.NORM_SLAB - 1) // K.NORM_SLAB
            assert n_slabs & (n_slabs - 1) == 0, "tensor parallelism needs a power-of-two number of 8-row slabs per rank"
            roots = _all_gather(dg)
            while len(roots) > 1:
                roots = [roots[i] + roots[i + 1] if i + 1 < len(roots) else roots[i] for i in range(0, len(roots), 2)]
            dg = roots[0]
            if _TP.rank != 0:
                need_dg = False
        if need_dg:
            if ctx.slot is not None and ctx.slot.buf is not None:
                if ctx.slot.take():
                    ctx.slot.buf.copy_(dg)
                else:
                    ctx.slot.buf.add_(dg)
            else:
                gm = dg.to(ctx.master_dtype)
        return dx.view(ctx.shape), gm, None, None, None, None


def rms_norm(x, master, w=None, slot=None, eps=1e-5, tp_heads=0):
    """``tp_heads``: under tensor parallelism, the rows of ``x`` are (token, head) pairs with this many local heads per
    token (the heads are split over the group); 0 = the rows are this rank's tokens."""
    if master is None:
        return RMSNormFn.apply(x, None, None, None, eps)
    return RMSNormFn.apply(x, master, master if w is None else w, slot, eps, tp_heads)


class SwiGLUFn(Function):
    @staticmethod
    def forward(ctx, gu):
        g2 = _flat2d(gu).contiguous()
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return K.swiglu_fwd(g2).view(*gu.shape[:-1], gu.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dh):
        (g2,) = ctx.saved_tensors
        return K.swiglu_bwd(g2, _flat2d(dh).contiguous()).view(ctx.shape)


def swiglu(gate_up):
    return SwiGLUFn.apply(gate_up)


# Activation checkpointing recomputes a block's forward pass inside the backward pass. On a CPU the attention forward is
# by far the most expensive part of that recomputation and its results (output and log-sum-exp rows) are small next to
# the activations the checkpoint drops, so a replay on a CPU may keep them: `cpu_attention_checkpoint_contexts` is a
# `context_fn` for torch.utils.checkpoint - the first context records the attention results of the original forward pass,
# the second hands them out, in call order, to the recomputation. Bit-neutral: the recomputation would produce the same
# values (reference: repop's cpu_attention_checkpoint_contexts, src/pretrain/parallel/parallelize_llama3_repop.py:118-124).
_attn_cache: dict = {"mode": None, "store": None, "hits": 0}


class _AttnCacheCtx:
    def __init__(self, mode, store):
        self.mode, self.store, self.prev = mode, store, None

    def __enter__(self):
        self.prev = (_attn_cache["mode"], _attn_cache["store"])
        _attn_cache["mode"], _attn_cache["store"] = self.mode, self.store
        if self.mode == "replay":
            self.store["next"] = 0
        return self

    def __exit__(self, *exc):
        _attn_cache["mode"], _attn_cache["store"] = self.prev
        return False


def cpu_attention_checkpoint_contexts():
    store = {"results": [], "next": 0}
    return _AttnCacheCtx("record", store), _AttnCacheCtx("replay", store)


def _attn_fwd_cached(qk, q2, B, T, H, Hkv, D, window, int8_pv):
    mode, store = _attn_cache["mode"], _attn_cache["store"]
    if mode == "replay" and not qk.is_cuda and store["next"] < len(store["results"]):
        out = store["results"][store["next"]]
        store["next"] += 1
        _attn_cache["hits"] += 1
        return out
    out = K.attn_fwd(qk, q2, B, T, H, Hkv, D, window, int8_pv)
    if mode == "record" and not qk.is_cuda:
        store["results"].append(out)
    return out


class AttentionFn(Function):
    """(gain-free QK-norm) -> RoPE -> causal / sliding-window flash attention on a packed qkv
    activation [B, T, (H + 2 Hkv) D]; returns [B, T, H D]."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, H, Hkv, D, window, qk_norm, eps, int8_pv=False):
        B, T, _ = qkv.shape
        q2 = qkv.reshape(B * T, -1)
        qk, rstd = K.qknorm_rope_fwd(q2, cos, sin, H + Hkv, D, T, qk_norm, eps)
        # int8 P V: quantised forward, straight-through (float shadow) backward through the ordinary kernels
        O, lse = _attn_fwd_cached(qk, q2, B, T, H, Hkv, D, window, int8_pv)
        ctx.save_for_backward(q2, qk, rstd, O, lse, cos, sin)
        ctx.cfg = (B, T, H, Hkv, D, window, qk_norm)
        return O.view(B, T, H * D)

    @staticmethod
    def backward(ctx, dO):
        q2, qk, rstd, O, lse, cos, sin = ctx.saved_tensors
        B, T, H, Hkv, D, window, qk_norm = ctx.cfg
        dO2 = dO.reshape(B * T, H * D)
        if not dO2.is_contiguous():
            dO2 = dO2.contiguous()
        dqk = torch.empty_like(qk)
        dqkv = torch.empty_like(q2)
        K.attn_bwd(qk, q2, O, dO2, lse, dqk, dqkv, B, T, H, Hkv, D, window)
        K.qknorm_rope_bwd(dqk, q2, rstd, dqkv, cos, sin, H + Hkv, D, T, qk_norm)
        return dqkv.view(B, T, -1), None, None, None, None, None, None, None, None, None


def attention(qkv, cos, sin, H, Hkv, D, window, qk_norm, eps, int8_pv=False):
    return AttentionFn.apply(qkv, cos, sin, H, Hkv, D, window, qk_norm, eps, int8_pv)


class EmbeddingFn(Function):
    @staticmethod
    def forward(ctx, ids, master, table, slot):
        ctx.save_for_backward(ids)
        ctx.slot = slot
        ctx.tshape = table.shape
        ctx.master_dtype = master.dtype
        return K.embedding_fwd(ids, table).view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        dy2 = _flat2d(dy).contiguous()
        if _TP is not None:
            # rows accumulate in ascending token position over the WHOLE micro-batch: rank 0 gets every row and runs the
            # one deterministic scatter
            dy2 = tp_gather_rows(dy2)
            ids = tp_gather_rows(ids.reshape(-1))
            if _TP.rank != 0:
                return None, None, None, None
        if ctx.slot is not None and ctx.slot.buf is not None:
            ctx.slot.zero_if_first()  # rows of tokens that do not occur must read zero
            K.embedding_bwd(dy2, ids, ctx.slot.buf, True)
            return None, None, None, None
        dW = torch.zeros(ctx.tshape, dtype=torch.float32, device=dy.device)
        K.embedding_bwd(dy2, ids, dW, False)
        return None, dW.to(ctx.master_dtype), None, None


def embedding(ids, master, table=None, slot=None):
    return EmbeddingFn.apply(ids, master, master if table is None else table, slot)


class FusedCEZLossFn(Function):
    """Mean cross-entropy and z-loss (coeff * mean lse^2) over rows with label >= 0.

    The gradient w.r.t. the logits is produced in the forward pass, in place of the logits, already
    multiplied by ``grad_scale`` (1/accum): the incoming gradients of both outputs must equal that
    scale, which is what ``(ce + z) * (1/accum)`` gives. One log-sum-exp per row, fixed-order row
    reduction, mean by multiplication with the host reciprocal 1/N
    (reference src/pretrain/model/fused_loss.py:40-104)."""

    @staticmethod
    def forward(ctx, logits, labels, z_coeff, grad_scale):
        l2 = _flat2d(logits)
        assert l2.is_contiguous()
        lab = labels.reshape(-1).contiguous()
        n_valid = lab.numel() * (_TP.size if _TP is not None else 1)  # callers with ignored rows pass n via grad_scale themselves
        inv_n = 1.0 / n_valid
        need_grad = logits.requires_grad
        ce_rows, lse_rows = K.ce_zloss_(l2, lab, z_coeff, inv_n * grad_scale, write_grad=need_grad)
        if _TP is not None:  # the means run over every row of the micro-batch in the unsplit order
            ce_rows, lse_rows = tp_gather_rows(ce_rows), tp_gather_rows(lse_rows)
        ce = K.det_sum(ce_rows, False, inv_n)
        z = K.det_sum(lse_rows, True, inv_n) * z_coeff
        # The logits buffer now holds the gradient. It is an activation nobody else saved (the
        # vocabulary projection keeps its input and weight, not its output), so overwriting it is safe.
        ctx.grad_buf = l2 if need_grad else None
        ctx.shape = logits.shape
        return ce.reshape(()), z.reshape(())

    @staticmethod
    def backward(ctx, dce, dz):
        g = ctx.grad_buf
        ctx.grad_buf = None
        return (g.view(ctx.shape) if g is not None else None), None, None, None


def fused_ce_z_loss(logits, labels, z_coeff: float, grad_scale: float = 1.0):
    ce, z = FusedCEZLossFn.apply(logits, labels, float(z_coeff), float(grad_scale))
    return ce, z


class QuantLinearFn(Function):
    """W8A8 quantisation-aware linear layer: activations quantised per tensor, weights per output channel, the
    product taken exactly in int32 on the int8 tensor cores, one fp32 dequantisation, straight-through backward.
    ``step`` is the per-channel step size (learned for ``lsq``; derived from the weights for ``absmax``, in which
    case ``learn_step`` is false and no step gradient is produced).
    (reference roles: repop.qat.lsq.LSQQuantizedLinear / repop.qat.QuantizedLinear built by
    src/pretrain/model/modules/_linear.py:31-65)"""

    @staticmethod
    def forward(ctx, x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache, hadamard=False):
        x2 = _flat2d(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        xq, sa = K.quant_act(x2, qmax_a)
        key = (K.weight_epoch, x2.dtype)
        if cache is not None and K.weight_epoch is not None and cache.get("key") == key:
            wq, w_hat = cache["wq"], cache["w_hat"]
        else:
            wq, w_hat = K.quant_weight(w, step, qmax_w, x2.dtype)
            if cache is not None and K.weight_epoch is not None:
                cache.update(key=key, wq=wq, w_hat=w_hat)
        y = K.gemm_i8(xq, wq, sa, step, x2.dtype, _flat2d(residual) if residual is not None else None)
        ctx.save_for_backward(xq, sa, w_hat, w, step)
        ctx.slot_w, ctx.slot_s = slot_w, slot_s
        ctx.has_res = residual is not None
        ctx.in_shape = x.shape
        ctx.cfg = (qmax_w, learn_step, master_w.dtype, None if master_s is None else master_s.dtype)
        ctx.hadamard = bool(hadamard)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xq, sa, w_hat, w, step = ctx.saved_tensors
        qmax_w, learn_step, w_dtype, s_dtype = ctx.cfg
        dy2 = _flat2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        B = K.HADAMARD_BLOCK
        if ctx.hadamard and dy2.shape[0] % B == 0 and dy2.shape[1] % B == 0:
            # both straight-through GEMMs on the int8 tensor cores, operands Hadamard-rotated along the contraction index
            dx = None
            if ctx.needs_input_grad[0]:
                dx = K.ste_matmul_hadamard(dy2, w_hat.t().contiguous()).to(dy2.dtype).view(ctx.in_shape)
            G = K.ste_matmul_hadamard(dy2.t().contiguous(), K.i8_widen(xq, torch.float32).t().contiguous())
        else:
            dx = K.gemm(dy2, w_hat, b_mn=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
            # dL/dw_hat = dy^T x_hat with x_hat = xq * sa: the integers are exact in bf16, the step is applied afterwards
            G = K.gemm(dy2, K.i8_widen(xq, dy2.dtype), a_mn=True, b_mn=True, epi=K.EPI_STORE_F32)
        N, Kd = w.shape
        gs = 1.0 / math.sqrt(float(Kd) * float(qmax_w))
        use_slot = ctx.slot_w is not None and ctx.slot_w.buf is not None
        if use_slot:
            ctx.slot_w.zero_if_first()
        dW = ctx.slot_w.buf if use_slot else torch.zeros((N, Kd), dtype=torch.float32, device=w.device)
        ds = None
        if learn_step:
            s_slot = ctx.slot_s is not None and ctx.slot_s.buf is not None
            if s_slot:
                ctx.slot_s.zero_if_first()
            ds = ctx.slot_s.buf if s_slot else torch.zeros(N, dtype=torch.float32, device=w.device)
        # a fixed (absmax) step never clips, so its mask bound is one grid point wider than the grid
        K.lsq_bwd_(G, w, step, sa, qmax_w if learn_step else qmax_w + 1, gs, dW, ds)
        gw = None if use_slot else dW.to(w_dtype)
        gsm = None
        if learn_step and not (ctx.slot_s is not None and ctx.slot_s.buf is not None):
            gsm = ds.to(s_dtype)
        return dx, gw, None, None, gsm, None, None, (dy if ctx.has_res else None), None, None, None, None, None


class TpQuantLinearFn(Function):
    """The W8A8 layer under tensor parallelism. ``mode`` "col": ``x`` is this rank's token rows, the rank produces the output
    features ``parts[rank]`` (ranges of W's rows) for all tokens. ``mode`` "row": ``x`` holds the input features
    ``parts[rank]`` (one range of W's columns) of all tokens, the result comes back as this rank's token rows (+ residual).
    The activation step is the absmax of the WHOLE activation, as in the unsplit layer, so the operand is gathered before it
    is quantised; integer products are exact, and the float reductions (data gradient over all output features, weight
    gradient over all tokens, step gradient over all input features) each run unsplit on the rank that owns the result:
    for "row" the weight and step gradients are split by OUTPUT rows, which needs no further exchange."""

    @staticmethod
    def forward(ctx, x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache, mode, parts):
        st = _TP
        x2 = _flat2d(x).contiguous()
        x_full = tp_gather_rows(x2) if mode == "col" else tp_gather_cols(x2, [[c] for c in parts], w.shape[1])
        xq, sa = K.quant_act(x_full, qmax_a)
        key = (K.weight_epoch, x2.dtype)
        if cache is not None and K.weight_epoch is not None and cache.get("key") == key:
            wq, w_hat = cache["wq"], cache["w_hat"]
        else:
            wq, w_hat = K.quant_weight(w, step, qmax_w, x2.dtype)
            if cache is not None and K.weight_epoch is not None:
                cache.update(key=key, wq=wq, w_hat=w_hat)
        if mode == "col":
            mine = parts[st.rank]
            y = torch.cat([K.gemm_i8(xq, wq[a:b], sa, step[a:b].contiguous(), x2.dtype) for a, b in mine], 1)
        else:
            res = _flat2d(residual).contiguous() if residual is not None else None
            y = K.gemm_i8(xq[st.rows(xq.shape[0])], wq, sa, step, x2.dtype, res)
        ctx.save_for_backward(xq, sa, w_hat, w, step)
        ctx.slot_w, ctx.slot_s = slot_w, slot_s
        ctx.has_res = residual is not None
        ctx.cfg = (qmax_w, learn_step, mode, parts)
        return y

    @staticmethod
    def backward(ctx, dy):
        xq, sa, w_hat, w, step = ctx.saved_tensors
        qmax_w, learn_step, mode, parts = ctx.cfg
        st = _TP
        dy = dy.contiguous()
        N, Kd = w.shape
        if mode == "col":
            rows_w = parts[st.rank]                       # this rank's output features: their gradient rows
            dy_mine = dy                                  # [M, n_t], all tokens
            dy_full = tp_gather_cols(dy, parts, N)
            dx = K.gemm(dy_full[st.rows(dy_full.shape[0])].contiguous(), w_hat, b_mn=True)
        else:
            dy_full = tp_gather_rows(dy)                  # [M, N]
            a, b = parts[st.rank]
            dx = K.gemm(dy_full, w_hat[:, a:b], b_mn=True)
            rows_w = [st.split(N)]
            dy_mine = dy_full[:, rows_w[0][0]:rows_w[0][1]].contiguous()
        G = K.gemm(dy_mine, K.i8_widen(xq, dy.dtype), a_mn=True, b_mn=True, epi=K.EPI_STORE_F32)  # [n_t, K], every token
        gs = 1.0 / math.sqrt(float(Kd) * float(qmax_w))
        slot_w = _tp_slot(ctx.slot_w)
        slot_s = _tp_slot(ctx.slot_s) if learn_step else None
        off = 0
        for a, b in rows_w:
            K.lsq_bwd_(G[off:off + (b - a)], w[a:b], step[a:b].contiguous(), sa, qmax_w if learn_step else qmax_w + 1, gs,
                       slot_w.buf[a:b], slot_s.buf[a:b] if learn_step else None)
            off += b - a
        return dx, None, None, None, None, None, None, (dy if ctx.has_res else None), None, None, None, None, None, None


def tp_quant_linear(x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache, mode, parts):
    return TpQuantLinearFn.apply(x, master_w, master_w if w is None else w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a,
                                 learn_step, cache, mode, parts)


def quant_linear(x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache=None, hadamard=False):
    return QuantLinearFn.apply(x, master_w, master_w if w is None else w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a,
                               learn_step, cache, hadamard)
