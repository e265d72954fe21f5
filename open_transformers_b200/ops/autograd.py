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

    __slots__ = ("buf", "fresh", "written")

    def __init__(self, buf: torch.Tensor | None = None):
        self.buf = buf
        self.fresh = False
        self.written = False

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


class LinearFn(Function):
    """y = x W^T (+ residual). ``master`` is the fp32 parameter autograd knows about, ``w`` the
    compute-dtype weight actually multiplied (the same tensor in fp32 runs)."""

    @staticmethod
    def forward(ctx, x, master, w, slot, residual):
        x2 = _flat2d(x)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if residual is not None:
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


class RMSNormFn(Function):
    @staticmethod
    def forward(ctx, x, master, w, slot, eps):
        x2 = _flat2d(x).contiguous()
        y, rstd = K.rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, rstd, w if w is not None else x2.new_empty(0))
        ctx.has_w = w is not None
        ctx.slot = slot
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
        if need_dg:
            if ctx.slot is not None and ctx.slot.buf is not None:
                if ctx.slot.take():
                    ctx.slot.buf.copy_(dg)
                else:
                    ctx.slot.buf.add_(dg)
            else:
                gm = dg.to(ctx.master_dtype)
        return dx.view(ctx.shape), gm, None, None, None


def rms_norm(x, master, w=None, slot=None, eps=1e-5):
    if master is None:
        return RMSNormFn.apply(x, None, None, None, eps)
    return RMSNormFn.apply(x, master, master if w is None else w, slot, eps)


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


class AttentionFn(Function):
    """(gain-free QK-norm) -> RoPE -> causal / sliding-window flash attention on a packed qkv
    activation [B, T, (H + 2 Hkv) D]; returns [B, T, H D]."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, H, Hkv, D, window, qk_norm, eps, int8_pv=False):
        B, T, _ = qkv.shape
        q2 = qkv.reshape(B * T, -1)
        qk, rstd = K.qknorm_rope_fwd(q2, cos, sin, H + Hkv, D, T, qk_norm, eps)
        # int8 P V: quantised forward, straight-through (float shadow) backward through the ordinary kernels
        O, lse = K.attn_fwd(qk, q2, B, T, H, Hkv, D, window, int8_pv)
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
        n_valid = lab.numel()  # callers with ignored rows pass n via grad_scale themselves
        inv_n = 1.0 / n_valid
        need_grad = logits.requires_grad
        ce_rows, lse_rows = K.ce_zloss_(l2, lab, z_coeff, inv_n * grad_scale, write_grad=need_grad)
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
    def forward(ctx, x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache):
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
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xq, sa, w_hat, w, step = ctx.saved_tensors
        qmax_w, learn_step, w_dtype, s_dtype = ctx.cfg
        dy2 = _flat2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
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
        return dx, gw, None, None, gsm, None, None, (dy if ctx.has_res else None), None, None, None, None


def quant_linear(x, master_w, w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a, learn_step, cache=None):
    return QuantLinearFn.apply(x, master_w, master_w if w is None else w, slot_w, master_s, step, slot_s, residual, qmax_w, qmax_a,
                               learn_step, cache)
