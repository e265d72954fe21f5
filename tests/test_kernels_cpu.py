"""CPU twins against plain PyTorch references, plus the invariances the hashed contract relies on."""
import math

import pytest
import torch
import torch.nn.functional as Fn

from open_transformers_b200.models import fused_ce_z_loss, streaming_head_loss
from open_transformers_b200.ops import autograd as A
from open_transformers_b200.ops import functional as K


def test_gemm_variants_match_matmul_and_are_order_exact():
    g = torch.Generator().manual_seed(0)
    A_, B_ = torch.randn(33, 70, generator=g), torch.randn(21, 70, generator=g)
    ref = A_ @ B_.t()
    for a_mn, b_mn in ((0, 0), (0, 1), (1, 1), (1, 0)):
        out = K.gemm(A_.t().contiguous() if a_mn else A_, B_.t().contiguous() if b_mn else B_, a_mn=bool(a_mn), b_mn=bool(b_mn))
        assert torch.allclose(out, ref, atol=1e-4)
        assert torch.equal(out, K.gemm(A_, B_))  # the storage order never changes the bits
    # one ascending-k fma chain per element
    acc = torch.zeros((), dtype=torch.float64)
    a, b = A_[3].double(), B_[5].double()
    chain = 0.0
    import numpy as np
    c = np.float32(0)
    for k in range(70):
        c = np.float32(np.float64(np.float32(A_[3, k])) * np.float64(np.float32(B_[5, k])) + np.float64(c))
    assert abs(float(out[3, 5]) - float(c)) <= 1e-6  # fma in fp64 then one rounding == fused multiply-add


def test_rmsnorm_swiglu_match_torch():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 256, generator=g, requires_grad=True)
    w = (1 + 0.1 * torch.randn(256, generator=g)).requires_grad_(True)
    y = A.rms_norm(x, w, eps=1e-5)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(y, ref, atol=1e-5)
    gy = torch.randn(9, 256, generator=g)
    gx, gw = torch.autograd.grad(y, (x, w), gy)
    rx, rw = torch.autograd.grad(ref, (x, w), gy)
    assert torch.allclose(gx, rx, atol=1e-5) and torch.allclose(gw, rw, atol=1e-4)
    gu = torch.randn(7, 128, generator=g, requires_grad=True)
    h = A.swiglu(gu)
    a, b = gu.chunk(2, -1)
    href = Fn.silu(a) * b
    assert torch.allclose(h, href, atol=1e-6)
    gg = torch.randn(7, 64, generator=g)
    assert torch.allclose(torch.autograd.grad(h, gu, gg)[0], torch.autograd.grad(href, gu, gg)[0], atol=1e-5)


@pytest.mark.parametrize("window,T,Hkv", [(0, 160, 2), (64, 300, 1)])
def test_attention_matches_sdpa(window, T, Hkv):
    g = torch.Generator().manual_seed(2)
    B, H, D = 2, 2, 64
    qkv = torch.randn(B, T, (H + 2 * Hkv) * D, generator=g, requires_grad=True)
    cos, sin = K.rope_tables(T, D, 10000.0, "cpu")
    o = A.attention(qkv, cos, sin, H, Hkv, D, window, True, 1e-5)
    q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)

    def norm_rope(t, n):
        t = t.view(B, T, n, D)
        t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5)
        te, to = t[..., 0::2], t[..., 1::2]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack([te * c - to * s, te * s + to * c], -1).flatten(-2)

    qr, kr = norm_rope(q, H).transpose(1, 2), norm_rope(k, Hkv).transpose(1, 2).repeat_interleave(H // Hkv, 1)
    vr = v.view(B, T, Hkv, D).transpose(1, 2).repeat_interleave(H // Hkv, 1)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = (j <= i) & ((j > i - window) if window else True)
    ref = Fn.scaled_dot_product_attention(qr, kr, vr, attn_mask=mask).transpose(1, 2).reshape(B, T, H * D)
    assert torch.allclose(o, ref, atol=2e-5)
    go = torch.randn(B, T, H * D, generator=g)
    assert torch.allclose(torch.autograd.grad(o, qkv, go)[0], torch.autograd.grad(ref, qkv, go)[0], atol=5e-5)


def test_fused_loss_matches_torch_and_streaming_head_is_bitwise_equal():
    g = torch.Generator().manual_seed(3)
    n, d, V = 48, 64, 256
    h = torch.randn(n, d, generator=g)
    W = (0.1 * torch.randn(V, d, generator=g)).requires_grad_(True)
    labels = torch.randint(0, V, (n,), generator=g)
    hq = h.clone().requires_grad_(True)
    logits = A.linear(hq, W)
    ce, z = fused_ce_z_loss(logits, labels, 1e-3)
    (ce + z).backward()
    ref_logits = h @ W.detach().t()
    lse = torch.logsumexp(ref_logits, -1)
    assert ce.item() == pytest.approx(Fn.cross_entropy(ref_logits, labels).item(), rel=1e-6)
    assert z.item() == pytest.approx(1e-3 * lse.pow(2).mean().item(), rel=1e-5)
    # streaming head: panels of 16 rows, same bytes for ce, z, dH and dW
    ce2, z2, dh2, dW2 = streaming_head_loss(h, W.detach(), labels, 1e-3, panel_rows=16)
    assert torch.equal(ce2, ce.detach()) and torch.equal(z2, z.detach())
    assert torch.equal(dh2, hq.grad) and torch.equal(dW2, W.grad)


def test_embedding_backward_is_sorted_segment_sum():
    g = torch.Generator().manual_seed(4)
    W = torch.randn(32, 16, generator=g, requires_grad=True)
    ids = torch.tensor([[3, 5, 3, 3], [5, 0, 31, 3]])
    x = A.embedding(ids, W)
    gy = torch.randn(2, 4, 16, generator=g)
    (gw,) = torch.autograd.grad(x, W, gy)
    want = torch.zeros_like(W)
    for pos, i in enumerate(ids.reshape(-1).tolist()):   # ascending token position per row: the pinned order
        want[i] = want[i] + gy.reshape(-1, 16)[pos]
    assert torch.equal(gw, want)


def test_det_math_against_libm():
    import ctypes

    from open_transformers_b200.ops.native import cpu_lib

    lib = cpu_lib()
    lib.otb_cpu_expf.restype = ctypes.c_float
    lib.otb_cpu_logf.restype = ctypes.c_float
    for x in (-50.0, -1.0, 0.0, 0.3, 10.0, 80.0):
        assert lib.otb_cpu_expf(ctypes.c_float(x)) == pytest.approx(math.exp(x), rel=3e-7)
    for x in (1e-20, 0.5, 1.0, 3.0, 1e20):
        assert lib.otb_cpu_logf(ctypes.c_float(x)) == pytest.approx(math.log(x), rel=3e-7, abs=1e-7)


def test_philox_init_is_split_invariant():
    a = torch.empty(1000)
    K.trunc_normal_(a, 0.02, 7, 0)
    b1, b2 = torch.empty(300), torch.empty(700)
    K.trunc_normal_(b1, 0.02, 7, 0)
    K.trunc_normal_(b2, 0.02, 7, 300)
    assert torch.equal(a, torch.cat([b1, b2]))
    assert a.abs().max() <= 0.04 + 1e-9 and abs(a.std().item() - 0.02 * 0.88) < 2e-3
    c = torch.empty(1000)
    K.trunc_normal_(c, 0.02, 8, 0)
    assert not torch.equal(a, c)
