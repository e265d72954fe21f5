"""sm_100a kernels against their CPU twins (bitwise where the contract is bit-exactness) and against
plain PyTorch fp32 references (tolerance) for the tensor-core family."""
import math

import pytest
import torch

from open_transformers_b200.ops import functional as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both(fn, *tensors, **kw):
    cpu = fn(*[t.cpu() if isinstance(t, torch.Tensor) else t for t in tensors], **kw)
    gpu = fn(*[t.to(DEV) if isinstance(t, torch.Tensor) else t for t in tensors], **kw)
    return cpu, gpu


def _eq(a, b, what):
    if isinstance(a, (tuple, list)):
        for i, (x, y) in enumerate(zip(a, b)):
            _eq(x, y, "%s[%d]" % (what, i))
        return
    if a is None:
        assert b is None
        return
    b = b.cpu()
    if not torch.equal(a, b):
        d = (a.float() - b.float()).abs()
        raise AssertionError("%s differs: max abs %.3e at %d of %d elements" % (what, d.max().item(), int((d > 0).sum()), d.numel()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(37, 256), (64, 2048), (5, 704)])
def test_rmsnorm_bitwise(dtype, rows, D):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, D, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    dy = torch.randn(rows, D, generator=g).to(dtype)
    for gain in (w, None):
        c, gq = _both(lambda x_, w_: K.rmsnorm_fwd(x_, w_, 1e-5), x, gain)
        _eq(c, gq, "rmsnorm_fwd")
        rstd = c[1]
        c2, g2 = _both(lambda dy_, x_, w_, r_: K.rmsnorm_bwd(dy_, x_, w_, r_, w_ is not None), dy, x, gain, rstd)
        _eq(c2, g2, "rmsnorm_bwd")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,do_norm", [(128, True), (64, True), (64, False)])
def test_qknorm_rope_bitwise(dtype, D, do_norm):
    g = torch.Generator().manual_seed(2)
    B, T, H, Hkv = 2, 48, 4, 2
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, generator=g).to(dtype)
    cos, sin = K.rope_tables(T, D, 10000.0, "cpu")
    c, gq = _both(lambda q, c_, s_: K.qknorm_rope_fwd(q, c_, s_, H + Hkv, D, T, do_norm, 1e-5), qkv, cos, sin)
    _eq(c[0], gq[0], "qknorm_rope_fwd")
    if do_norm:
        _eq(c[1], gq[1], "rstd")
    dout = torch.randn(B * T, (H + Hkv) * D, generator=g).to(dtype)

    def bwd(do_, q_, r_, c_, s_):
        din = torch.zeros_like(q_)
        return K.qknorm_rope_bwd(do_, q_, r_, din, c_, s_, H + Hkv, D, T, do_norm)

    c2, g2 = _both(bwd, dout, qkv, c[1], cos, sin)
    _eq(c2, g2, "qknorm_rope_bwd")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_bitwise(dtype):
    g = torch.Generator().manual_seed(3)
    gu = (3 * torch.randn(33, 2 * 704, generator=g)).to(dtype)
    dh = torch.randn(33, 704, generator=g).to(dtype)
    _eq(*_both(K.swiglu_fwd, gu), "swiglu_fwd")
    _eq(*_both(K.swiglu_bwd, gu, dh), "swiglu_bwd")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [1024, 8192 + 128])
def test_ce_zloss_bitwise(dtype, V):
    g = torch.Generator().manual_seed(4)
    rows = 19
    logits = (4 * torch.randn(rows, V, generator=g)).to(dtype)
    labels = torch.randint(0, V, (rows,), generator=g)
    labels[3] = -100

    def run(l_, lab_):
        l_ = l_.clone()
        ce, lse = K.ce_zloss_(l_, lab_, 1e-4, 1.0 / rows, True)
        return ce, lse, l_, K.det_sum(ce, False, 1.0 / rows), K.det_sum(lse, True, 1.0 / rows)

    c, gq = _both(run, logits, labels)
    _eq(c, gq, "ce_zloss")
    ref = torch.nn.functional.cross_entropy(logits.float(), labels, ignore_index=-100, reduction="none")
    assert torch.allclose(c[0], ref, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_bitwise(dtype):
    g = torch.Generator().manual_seed(5)
    V, D, n = 512, 256, 300
    table = torch.randn(V, D, generator=g).to(dtype)
    ids = torch.randint(0, 40, (n,), generator=g)
    dy = torch.randn(n, D, generator=g).to(dtype)
    _eq(*_both(K.embedding_fwd, ids, table), "embedding_fwd")

    def bwd(dy_, ids_):
        dW = torch.zeros(V, D, dtype=torch.float32, device=dy_.device)
        K.embedding_bwd(dy_, ids_, dW, True)
        K.embedding_bwd(dy_, ids_, dW, True)
        return dW

    _eq(*_both(bwd, dy, ids), "embedding_bwd")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K_", [(130, 70, 257), (256, 192, 64)])
def test_gemm_f32_bitwise(a_mn, b_mn, M, N, K_):
    g = torch.Generator().manual_seed(6)
    A = torch.randn(M, K_, generator=g)
    B = torch.randn(N, K_, generator=g)
    As = A.t().contiguous() if a_mn else A
    Bs = B.t().contiguous() if b_mn else B
    _eq(*_both(lambda a, b: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn), As, Bs), "gemm_f32")
    R = torch.randn(M, N, generator=g)
    _eq(*_both(lambda a, b, r: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_RESIDUAL, residual=r), As, Bs, R), "gemm_f32_res")

    def acc(a, b):
        out = torch.ones(M, N, device=a.device)
        return K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, epi=K.EPI_ACC_F32)

    _eq(*_both(acc, As, Bs), "gemm_f32_acc")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16_vs_reference(a_mn, b_mn):
    g = torch.Generator().manual_seed(7)
    M, N, K_ = 384, 520, 328
    A = torch.randn(M, K_, generator=g).bfloat16()
    B = torch.randn(N, K_, generator=g).bfloat16()
    ref = A.float() @ B.float().t()
    As = (A.t().contiguous() if a_mn else A).to(DEV)
    Bs = (B.t().contiguous() if b_mn else B).to(DEV)
    out = K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_STORE_F32).cpu()
    assert torch.allclose(out, ref, atol=2e-3, rtol=1e-4), (out - ref).abs().max()
    out2 = K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_STORE_F32).cpu()
    assert torch.equal(out, out2)
    # the other epilogues must agree with the fp32 store: bf16 store, residual add, fp32 accumulate (twice)
    o16 = K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn).cpu()
    assert torch.equal(o16, out.bfloat16())
    R = torch.randn(M, N, generator=g).bfloat16()
    ores = K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_RESIDUAL, residual=R.to(DEV)).cpu()
    assert torch.equal(ores, (out + R.float()).bfloat16())
    acc = torch.full((M, N), 0.5, device=DEV)
    K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, out=acc, epi=K.EPI_ACC_F32)
    K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, out=acc, epi=K.EPI_ACC_F32)
    assert torch.equal(acc.cpu(), (0.5 + out) + out)
    # a strided output view (weight-gradient slot inside a flat buffer) and a canary around it
    big = torch.full((M + 2, N + 16), 7.0, device=DEV)
    view = big[1:M + 1, 8:N + 8]
    K.gemm(As, Bs, a_mn=a_mn, b_mn=b_mn, out=view, epi=K.EPI_STORE_F32)
    assert torch.equal(view.cpu(), out)
    big[1:M + 1, 8:N + 8] = 7.0
    assert bool((big == 7.0).all())
    assert K.kernel_status(DEV) == 0


@pytest.mark.parametrize("D,window,T", [(64, 0, 200), (128, 0, 256), (64, 96, 320)])
def test_attention_f32_bitwise(D, window, T):
    g = torch.Generator().manual_seed(8)
    B, H, Hkv = 1, 4, 2
    qk = torch.randn(B * T, (H + Hkv) * D, generator=g)
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, generator=g)
    dO = torch.randn(B * T, H * D, generator=g)

    def run(qk_, qkv_, dO_):
        O, lse = K.attn_fwd(qk_, qkv_, B, T, H, Hkv, D, window)
        dqk, dqkv = torch.zeros_like(qk_), torch.zeros_like(qkv_)
        K.attn_bwd(qk_, qkv_, O, dO_, lse, dqk, dqkv, B, T, H, Hkv, D, window)
        return O, lse, dqk, dqkv[:, (H + Hkv) * D:].contiguous()

    _eq(*_both(run, qk, qkv, dO), "attention_f32")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_bf16_matches_tensor_core_model(a_mn, b_mn):
    """The tcgen05 accumulation (16 products + accumulator, 26-bit aligned truncation, truncated sum) is modelled
    exactly by the CPU twin: wide exponent spread, ragged K, every epilogue."""
    g = torch.Generator().manual_seed(11)
    M, N, K_ = 200, 136, 328
    A = (torch.randn(M, K_, generator=g) * torch.exp2(torch.randint(-12, 13, (M, K_), generator=g).float())).bfloat16()
    B = (torch.randn(N, K_, generator=g) * torch.exp2(torch.randint(-12, 13, (N, K_), generator=g).float())).bfloat16()
    As = A.t().contiguous() if a_mn else A
    Bs = B.t().contiguous() if b_mn else B
    _eq(*_both(lambda a, b: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_STORE_F32), As, Bs), "gemm_bf16 fp32 store")
    _eq(*_both(lambda a, b: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn), As, Bs), "gemm_bf16 bf16 store")
    R = torch.randn(M, N, generator=g).bfloat16()
    _eq(*_both(lambda a, b, r: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_RESIDUAL, residual=r), As, Bs, R), "gemm_bf16 residual")

    def acc(a, b):
        out = torch.full((M, N), 0.25, device=a.device)
        K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, epi=K.EPI_ACC_F32)
        return K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, epi=K.EPI_ACC_F32)

    _eq(*_both(acc, As, Bs), "gemm_bf16 accumulate")


@pytest.mark.parametrize("D,window,T", [(128, 0, 300), (64, 96, 384), (128, 192, 448), (128, 0, 640)])
def test_attention_bf16_bitwise_vs_twin(D, window, T):
    g = torch.Generator().manual_seed(12)
    B, H, Hkv = 1, 4, 2
    qk = torch.randn(B * T, (H + Hkv) * D, generator=g).bfloat16()
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, generator=g).bfloat16()
    dO = (0.5 * torch.randn(B * T, H * D, generator=g)).bfloat16()

    def run(qk_, qkv_, dO_):
        O, lse = K.attn_fwd(qk_, qkv_, B, T, H, Hkv, D, window)
        dqk, dqkv = torch.zeros_like(qk_), torch.zeros_like(qkv_)
        K.attn_bwd(qk_, qkv_, O, dO_, lse, dqk, dqkv, B, T, H, Hkv, D, window)
        return O, lse, dqk, dqkv[:, (H + Hkv) * D:].contiguous()

    _eq(*_both(run, qk, qkv, dO), "attention_bf16")
    assert K.kernel_status(DEV) == 0


@pytest.mark.parametrize("D,window,T", [(128, 0, 384), (64, 128, 512)])
def test_attention_bf16_vs_twin(D, window, T):
    g = torch.Generator().manual_seed(9)
    B, H, Hkv = 2, 4, 2
    qk = torch.randn(B * T, (H + Hkv) * D, generator=g).bfloat16()
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, generator=g).bfloat16()
    dO = (0.5 * torch.randn(B * T, H * D, generator=g)).bfloat16()

    def run(qk_, qkv_, dO_):
        O, lse = K.attn_fwd(qk_, qkv_, B, T, H, Hkv, D, window)
        dqk, dqkv = torch.zeros_like(qk_), torch.zeros_like(qkv_)
        K.attn_bwd(qk_, qkv_, O, dO_, lse, dqk, dqkv, B, T, H, Hkv, D, window)
        return O.float(), lse, dqk.float(), dqkv[:, (H + Hkv) * D:].float()

    c, gq = _both(run, qk, qkv, dO)
    for name, a, b in zip(("O", "lse", "dqk", "dv"), c, gq):
        err = (a - b.cpu()).abs().max().item()
        assert err < 0.04 * max(1.0, a.abs().max().item()), (name, err)
    assert K.kernel_status(DEV) == 0


def test_tree_digest_matches_host():
    from open_transformers_b200.train import state_hash as SH

    g = torch.Generator().manual_seed(10)
    for n in (0, 5, 1024, 1025, 300_000, 5_000_000):
        t = torch.randn(n, generator=g)
        assert SH.tree_digest_tensor(t) == SH.tree_digest_tensor(t.to(DEV)), n


@pytest.mark.parametrize("S,R", [(4, 1), (2, 2), (8, 1), (2, 3), (1, 7)])
def test_grad_reduce_gpu_equals_cpu_fold_in_any_launch_order(S, R):
    """The fused reduction (ascending shard fold, replica pair tree, squared-norm partials) against the CPU fold, bit for
    bit; and the same chunks launched in reversed and in shuffled order (the bucketed launches of the overlapped path):
    every chunk is owned by one block, so the order of the blocks must not reach the bytes."""
    import ctypes

    import numpy as np

    from open_transformers_b200.ops.native import I, P, cpu_lib, cuda_lib, stream_ptr
    from open_transformers_b200.train.engine import _ptr_array

    g = torch.Generator().manual_seed(S * 10 + R)
    n = 5 * 8192 + 1000
    starts = np.arange(0, n, 8192, dtype=np.int64)
    lens = np.minimum(8192, n - starts).astype(np.int32)
    srcs_cpu = [torch.randn(n, generator=g) * 1e-3 for _ in range(S * R)]
    out_cpu, sos_cpu = torch.zeros(n), torch.zeros(len(starts))
    cs, cl = torch.from_numpy(starts), torch.from_numpy(lens)
    assert cpu_lib().otb_cpu_grad_reduce(_ptr_array([t.data_ptr() for t in srcs_cpu]), I(S), I(R), P(cs), P(cl), I(len(starts)), P(out_cpu), P(sos_cpu)) == 0
    srcs = [t.to(DEV) for t in srcs_cpu]
    ptrs = _ptr_array([t.data_ptr() for t in srcs])
    csd, cld = cs.to(DEV), cl.to(DEV)
    lib = cuda_lib()
    out, sos = torch.zeros(n, device=DEV), torch.zeros(len(starts), device=DEV)
    assert lib.otb_grad_reduce(ptrs, I(S), I(R), P(csd), P(cld), I(len(starts)), P(out), P(sos), stream_ptr()) == 0
    _eq(out_cpu, out, "reduced gradient")
    _eq(sos_cpu, sos, "chunk partials")
    for order in (list(range(len(starts)))[::-1], [3, 0, 5, 1, 4, 2]):
        ids = torch.tensor(order, dtype=torch.int32, device=DEV)
        out2, sos2 = torch.full((n,), 9.0, device=DEV), torch.full((len(starts),), 9.0, device=DEV)
        assert lib.otb_grad_reduce_ids(ptrs, I(S), I(R), P(csd), P(cld), P(ids), I(len(order)), P(out2), P(sos2), stream_ptr()) == 0
        _eq(out_cpu, out2, "reduced gradient, launch order %s" % order)
        _eq(sos_cpu, sos2, "chunk partials, launch order %s" % order)
    del ctypes


def test_gpu_hadamard_int8_product_bitwise_vs_cpu():
    """rotation (IEEE adds), row statistics, quantiser and the tcgen05 kind::i8 GEMM give the CPU twin's bits"""
    g = torch.Generator().manual_seed(8)
    a, b = torch.randn(256, 384, generator=g), torch.randn(136, 384, generator=g).bfloat16()
    a[5, 100] = 90.0
    cpu, gpu = _both(lambda a_, b_: K.ste_matmul_hadamard(a_, b_), a, b)
    assert torch.equal(cpu, gpu.cpu()), "%d elements differ" % int((cpu != gpu.cpu()).sum())
    assert K.kernel_status("cuda") == 0


def test_adamw_amsgrad_gpu_equals_cpu_bitwise():
    """the AdamW kernel with the running maximum of the second moment: three steps on the GPU and on the CPU twin, bit for bit"""
    from open_transformers_b200.optim.adamw import DeterministicAdamW

    g = torch.Generator().manual_seed(9)
    w0 = torch.randn(5, 8192 + 40, generator=g)
    grads = [torch.randn(5, 8192 + 40, generator=g) * s for s in (1.0, 0.1, 3.0)]
    out = {}
    for dev in ("cpu", DEV):
        p = torch.nn.Parameter(w0.clone().to(dev))
        opt = DeterministicAdamW([p], lr=3e-3, weight_decay=0.1, amsgrad=True)
        for gr in grads:
            p.grad = gr.clone().to(dev)
            opt.step()
        out[dev] = (p.detach().cpu(), opt.state[p]["exp_avg_sq"].cpu(), opt.state[p]["max_exp_avg_sq"].cpu())
    for a, b, what in zip(out["cpu"], out[DEV], ("parameter", "second moment", "its running maximum")):
        _eq(a, b, what)


def test_gemm_and_attention_bytes_do_not_depend_on_the_launch_order():
    """Permuted launch order: with the test-only rotation each CTA takes over another CTA's share of the tiles (GEMM: the
    persistent workers; attention: the query tiles / key blocks of the grid's x axis). Every output element is owned by one
    CTA and summed in a fixed order, so the bytes must not move; a difference would be a race or an order that follows the
    schedule."""
    from open_transformers_b200.ops.native import cuda_lib

    lib = cuda_lib()
    g = torch.Generator().manual_seed(21)
    M, N, K_ = 1504, 1104, 712                      # 12 x 9 tiles, ragged edges; row sizes are multiples of 16 bytes
    A = torch.randn(M, K_, generator=g).bfloat16().to(DEV)
    Bm = torch.randn(N, K_, generator=g).bfloat16().to(DEV)
    At = A.t().contiguous()
    B_, T, H, Hkv, D = 2, 640, 4, 2, 128
    qk = torch.randn(B_ * T, (H + Hkv) * D, generator=g).bfloat16().to(DEV)
    qkv = torch.randn(B_ * T, (H + 2 * Hkv) * D, generator=g).bfloat16().to(DEV)
    dO = (0.5 * torch.randn(B_ * T, H * D, generator=g)).bfloat16().to(DEV)

    def everything():
        acc = torch.full((M, N), 0.5, device=DEV)
        K.gemm(A, Bm, out=acc, epi=K.EPI_ACC_F32)
        outs = [K.gemm(A, Bm), K.gemm(A, Bm, epi=K.EPI_STORE_F32), K.gemm(At, Bm, a_mn=True), acc]
        for window in (0, 192):
            O, lse = K.attn_fwd(qk, qkv, B_, T, H, Hkv, D, window)
            dqk, dqkv = torch.zeros_like(qk), torch.zeros_like(qkv)
            K.attn_bwd(qk, qkv, O, dO, lse, dqk, dqkv, B_, T, H, Hkv, D, window)
            outs += [O, lse, dqk, dqkv]
        torch.cuda.synchronize()
        return [o.clone() for o in outs]

    base = everything()
    try:
        for rot in (1, 5, 37):
            assert lib.otb_set_cta_rotation(rot) == 0 and lib.otb_set_attn_rotation(rot) == 0
            for i, (a, b) in enumerate(zip(base, everything())):
                assert torch.equal(a, b), "output %d moved under rotation %d" % (i, rot)
    finally:
        assert lib.otb_set_cta_rotation(0) == 0 and lib.otb_set_attn_rotation(0) == 0
    assert K.kernel_status(DEV) == 0
