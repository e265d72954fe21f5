"""Shape sweeps of the CPU twins against plain PyTorch fp32 references, in both arithmetic families (fp32: one fused
multiply-add chain per element; bf16: the tensor-core accumulation model): odd sizes, tile tails, window edges, grouped
heads, repeated ids. The twins are what the GPU kernels are compared with bit for bit, so their own correctness is pinned
here, against independent arithmetic."""
import pytest
import torch
import torch.nn.functional as Fn

from open_transformers_b200.ops import autograd as A
from open_transformers_b200.ops import functional as K

TOL = {torch.float32: dict(rtol=1e-4, atol=1e-4), torch.bfloat16: dict(rtol=3e-2, atol=3e-2)}


def _close(got, want, dtype, scale=1.0):
    t = TOL[dtype]
    err = (got.float() - want.float()).abs().max().item()
    ref = want.float().abs().max().item()
    assert err <= t["atol"] * scale + t["rtol"] * ref, (err, ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,Kd", [(1, 8, 8), (5, 24, 40), (129, 72, 136), (64, 264, 520), (130, 8, 1032)])
def test_gemm_shapes_and_epilogues(dtype, M, N, Kd):
    g = torch.Generator().manual_seed(M * 1000 + N)
    a = torch.randn(M, Kd, generator=g).to(dtype)
    b = (torch.randn(N, Kd, generator=g) * 0.1).to(dtype)
    r = torch.randn(M, N, generator=g).to(dtype)
    ref = a.float() @ b.float().t()
    _close(K.gemm(a, b), ref, dtype)
    _close(K.gemm(a, b.t().contiguous(), b_mn=True), ref, dtype)
    _close(K.gemm(a.t().contiguous(), b.t().contiguous(), a_mn=True, b_mn=True), ref, dtype)
    _close(K.gemm(a, b, epi=K.EPI_RESIDUAL, residual=r), ref + r.float(), dtype)
    acc = torch.full((M, N), 0.5)
    K.gemm(a, b, out=acc, epi=K.EPI_ACC_F32)
    _close(acc, ref + 0.5, dtype)
    store = torch.full((M, N), 7.0)
    K.gemm(a, b, out=store, epi=K.EPI_STORE_F32)
    _close(store, ref, dtype)
    assert store.dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,Hkv,T,D,window", [(1, 4, 1, 96, 64, 0), (2, 2, 2, 192, 128, 0), (1, 4, 2, 224, 64, 32), (1, 2, 1, 320, 128, 128),
                                                (1, 2, 2, 160, 64, 160), (1, 8, 2, 64, 32, 0)])
def test_attention_shapes_windows_and_grouping(dtype, B, H, Hkv, T, D, window):
    g = torch.Generator().manual_seed(T + D + window)
    qkv = (torch.randn(B, T, (H + 2 * Hkv) * D, generator=g) * 0.5).to(dtype).requires_grad_(True)
    cos, sin = K.rope_tables(T, D, 10000.0, "cpu")
    o = A.attention(qkv, cos, sin, H, Hkv, D, window, False, 1e-5)
    f = qkv.detach().float().requires_grad_(True)
    q, k, v = f.split([H * D, Hkv * D, Hkv * D], -1)

    def rope(t, n):
        t = t.view(B, T, n, D)
        te, to = t[..., 0::2], t[..., 1::2]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack([te * c - to * s, te * s + to * c], -1).flatten(-2)

    qr = rope(q, H).transpose(1, 2)
    kr = rope(k, Hkv).transpose(1, 2).repeat_interleave(H // Hkv, 1)
    vr = v.view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(H // Hkv, 1)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = (j <= i) & ((j > i - window) if window else True)
    ref = Fn.scaled_dot_product_attention(qr, kr, vr, attn_mask=mask).transpose(1, 2).reshape(B, T, H * D)
    _close(o, ref, dtype)
    go = torch.randn(B, T, H * D, generator=g)
    (got,) = torch.autograd.grad(o, qkv, go.to(dtype))
    (want,) = torch.autograd.grad(ref, f, go)
    _close(got, want, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D", [(1, 64), (7, 128), (33, 320), (130, 2048)])
def test_rmsnorm_and_swiglu_shapes(dtype, rows, D):
    g = torch.Generator().manual_seed(rows + D)
    x = torch.randn(rows, D, generator=g).to(dtype).requires_grad_(True)
    w32 = (1 + 0.1 * torch.randn(D, generator=g)).requires_grad_(True)
    y = A.rms_norm(x, w32, w32.detach().to(dtype) if dtype != torch.float32 else None, None, 1e-5)
    xf = x.detach().float().requires_grad_(True)
    wf = w32.detach().to(dtype).float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    _close(y, ref, dtype)
    gy = torch.randn(rows, D, generator=g)
    gx, gw = torch.autograd.grad(y, (x, w32), gy.to(dtype))
    rx, rw = torch.autograd.grad(ref, (xf, wf), gy.to(dtype).float())
    _close(gx, rx, dtype, scale=2.0)
    _close(gw, rw, dtype, scale=float(rows) ** 0.5)
    gu = torch.randn(rows, D, generator=g).to(dtype).requires_grad_(True)
    h = A.swiglu(gu)
    guf = gu.detach().float().requires_grad_(True)
    a, b = guf.chunk(2, -1)
    href = Fn.silu(a) * b
    _close(h, href, dtype)
    gh = torch.randn(rows, D // 2, generator=g)
    _close(torch.autograd.grad(h, gu, gh.to(dtype))[0], torch.autograd.grad(href, guf, gh.to(dtype).float())[0], dtype, scale=2.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,V", [(3, 128), (17, 1000), (64, 4104)])
def test_loss_rows_vocabulary_tails_and_gradient(dtype, n, V):
    g = torch.Generator().manual_seed(n + V)
    logits = (torch.randn(n, V, generator=g) * 3).to(dtype)
    labels = torch.randint(0, V, (n,), generator=g)
    lf = logits.float().requires_grad_(True)
    lse = torch.logsumexp(lf, -1)
    want = Fn.cross_entropy(lf, labels) + 1e-3 * lse.pow(2).mean()
    (gref,) = torch.autograd.grad(want, lf)
    work = logits.clone().requires_grad_(True)
    ce, z = A.fused_ce_z_loss(work, labels, 1e-3)
    (got,) = torch.autograd.grad(ce + z, work)
    assert float((ce + z).detach()) == pytest.approx(float(want.detach()), rel=2e-3 if dtype == torch.bfloat16 else 1e-5)
    _close(got, gref, dtype, scale=1.0 / n)


def test_embedding_backward_with_heavy_repeats_and_untouched_rows():
    g = torch.Generator().manual_seed(9)
    V, D = 97, 24
    W = torch.randn(V, D, generator=g, requires_grad=True)
    ids = torch.randint(0, 5, (3, 50), generator=g)            # five rows take all 150 positions
    ids[0, 0] = 96
    x = A.embedding(ids, W)
    gy = torch.randn(3, 50, D, generator=g)
    (gw,) = torch.autograd.grad(x, W, gy)
    want = torch.zeros_like(W)
    for pos, i in enumerate(ids.reshape(-1).tolist()):
        want[i] = want[i] + gy.reshape(-1, D)[pos]
    assert torch.equal(gw, want) and torch.count_nonzero(gw[5:96]) == 0


def test_fast_fp32_gemm_path_equals_the_plain_chain_loop_bit_for_bit():
    """the 4 x 16 micro-kernel (independent fused-multiply-add chains in SIMD lanes) against the one-element-at-a-time
    definition, over storage orders, epilogues, block tails and operand magnitudes"""
    from open_transformers_b200.ops.native import cpu_lib

    lib = cpu_lib()
    g = torch.Generator().manual_seed(0)

    def both(fn):
        lib.otb_cpu_gemm_set_plain(1)
        try:
            a = fn()
        finally:
            lib.otb_cpu_gemm_set_plain(0)
        return a, fn()

    for M, N, Kd in [(1, 1, 1), (1, 17, 5), (3, 16, 64), (5, 33, 129), (130, 70, 257), (4, 16, 16), (7, 15, 1000), (9, 48, 0)]:
        A = torch.randn(M, Kd, generator=g) * 10.0 ** torch.randint(-3, 3, (M, 1), generator=g).float()
        B, R, C0 = torch.randn(N, Kd, generator=g), torch.randn(M, N, generator=g), torch.randn(M, N, generator=g)
        for a_mn in (False, True):
            for b_mn in (False, True):
                aa, bb = (A.t().contiguous() if a_mn else A), (B.t().contiguous() if b_mn else B)
                if Kd == 0 and (a_mn or b_mn):
                    continue

                def acc():
                    c = C0.clone()
                    K.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, out=c, epi=K.EPI_ACC_F32)
                    return c

                def store():
                    c = torch.full((M, N), 3.0)
                    K.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, out=c, epi=K.EPI_STORE_F32)
                    return c

                for fn in (lambda: K.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn), lambda: K.gemm(aa, bb, a_mn=a_mn, b_mn=b_mn, epi=K.EPI_RESIDUAL, residual=R),
                           acc, store):
                    x, y = both(fn)
                    assert torch.equal(x, y), (M, N, Kd, a_mn, b_mn)


def test_fast_tensor_core_model_gemm_equals_the_plain_model_bit_for_bit():
    """bf16 family: the 16-columns-at-a-time restatement of the accumulation rule in vector arithmetic (exact fp32 products,
    power-of-two scaling, float -> int truncation, fp64 normalisation) against tcmodel::dot, over
    wide exponent spreads, sparse operands, near-cancellation, magnitudes at both ends of the fast path's range and beyond
    it (where it hands the element back to the plain routine), all epilogues and block tails"""
    from open_transformers_b200.ops.native import cpu_lib

    lib = cpu_lib()
    g = torch.Generator().manual_seed(1)

    def both(fn):
        lib.otb_cpu_gemm_set_plain(1)
        try:
            a = fn()
        finally:
            lib.otb_cpu_gemm_set_plain(0)
        return a, fn()

    def make(rows, Kd, mode):
        x = torch.randn(rows, Kd, generator=g)
        if mode == "spread":
            x = x * 2.0 ** torch.randint(-30, 30, (rows, Kd), generator=g).float()
        elif mode == "sparse":
            x = x * (torch.rand(rows, Kd, generator=g) < 0.3)
        elif mode == "cancel" and Kd > 1:
            half = x[:, 1::2].shape[1]
            x[:, 1::2] = -x[:, 0::2][:, :half] * (1 + 2.0 ** -7 * torch.randint(-1, 2, (rows, half), generator=g))
        elif mode in ("big", "small", "huge", "tiny", "subnormal"):
            x = x * 2.0 ** {"big": 45, "small": -55, "huge": 62, "tiny": -70, "subnormal": -130}[mode]
        return x.bfloat16()

    modes = ["normal", "spread", "sparse", "cancel", "big", "small", "huge", "tiny", "subnormal"]
    for M, N, Kd in [(1, 1, 1), (3, 17, 16), (5, 33, 40), (9, 70, 257), (2, 5, 1000)]:
        for i, ma in enumerate(modes):
            mb = modes[(i * 4 + M) % len(modes)]
            A, B = make(M, Kd, ma), make(N, Kd, mb)
            R, C0 = torch.randn(M, N, generator=g).bfloat16(), torch.randn(M, N, generator=g)

            def acc():
                c = C0.clone()
                K.gemm(A, B, out=c, epi=K.EPI_ACC_F32)
                return c

            for fn in (lambda: K.gemm(A, B), lambda: K.gemm(A, B.t().contiguous(), b_mn=True), lambda: K.gemm(A, B, epi=K.EPI_RESIDUAL, residual=R),
                       acc, lambda: K.gemm(A, B, epi=K.EPI_STORE_F32)):
                x, y = both(fn)
                same = torch.equal(torch.isnan(x), torch.isnan(y)) and torch.equal(torch.nan_to_num(x.float()), torch.nan_to_num(y.float()))
                assert same, (M, N, Kd, ma, mb)


@pytest.mark.parametrize("B,H,Hkv,T,D,window,qk_norm", [(1, 2, 1, 96, 64, 0, False), (2, 4, 2, 300, 64, 0, True), (1, 4, 1, 384, 128, 128, False),
                                                        (1, 2, 2, 260, 32, 64, True), (1, 4, 4, 130, 64, 32, False)])
def test_block_wise_bf16_attention_equals_the_plain_twin(B, H, Hkv, T, D, window, qk_norm):
    """the bf16 attention twins (forward: output and row statistic; backward) computed block by block through the lane-parallel accumulation kernel (scores and dP
    formed once per block pair, the three gradient chains continued in the plain routine's order) against the plain twin"""
    from open_transformers_b200.ops.native import cpu_lib

    lib = cpu_lib()
    g = torch.Generator().manual_seed(T + D)
    qkv = (torch.randn(B, T, (H + 2 * Hkv) * D, generator=g) * 0.7).bfloat16().requires_grad_(True)
    cos, sin = K.rope_tables(T, D, 10000.0, "cpu")
    go = torch.randn(B, T, H * D, generator=g).bfloat16()
    got = []
    for plain in (1, 0):
        lib.otb_cpu_gemm_set_plain(plain)
        try:
            o = A.attention(qkv, cos, sin, H, Hkv, D, window, qk_norm, 1e-5)
            (gq,) = torch.autograd.grad(o, qkv, go)
            q2 = qkv.detach().reshape(B * T, -1)
            rot, _ = K.qknorm_rope_fwd(q2, cos, sin, H + Hkv, D, T, qk_norm, 1e-5)
            _, lse = K.attn_fwd(rot, q2, B, T, H, Hkv, D, window, False)
        finally:
            lib.otb_cpu_gemm_set_plain(0)
        got.append((o.detach().clone(), gq.clone(), lse.clone()))
    assert torch.equal(got[0][0], got[1][0]) and torch.equal(got[0][1], got[1][1]) and torch.equal(got[0][2], got[1][2])
    assert float(got[1][1].float().abs().max()) > 0
