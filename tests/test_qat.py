"""int8 quantisation-aware training: the W8A8 layer against a plain PyTorch fp32 restatement of the same maths,
the warm-start switch, the step-size initialisation / refresh, and a whole run (train -> audit replay) with the
recipe flags on. GPU cases compare the sm_100a kernels (tcgen05 kind::i8 GEMM included) bit for bit with the CPU twins.
(reference test strategy: tests/distributed/test_lsq_fsdp_step.py:85-205)"""
import math

import pytest
import torch

from helpers import tiny_cfg
from open_transformers_b200.models.modules.core import Linear, QuantLinear, refresh_lsq_weight_scales, set_qat_active
from open_transformers_b200.ops import functional as K


def _layer(method, n_in=64, n_out=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    m = QuantLinear(n_in, n_out, method=method)
    with torch.no_grad():
        m.weight.copy_(torch.randn(n_out, n_in, generator=g) * 0.05)
        if method == "lsq":
            m.weight_scale.copy_(m.lsq_optimal_scale(m.weight))
    return m, g


@pytest.mark.parametrize("method", ["lsq", "absmax"])
def test_layer_matches_the_plain_formulas(method):
    m, g = _layer(method)
    x = torch.randn(3, 8, 64, generator=g, requires_grad=True)
    y = m(x)
    w = m.weight.detach()
    s = m.weight_scale.detach() if method == "lsq" else w.abs().amax(1) * (1.0 / 127)
    sa = x.detach().abs().max() * (1.0 / 127)
    xq = torch.clamp(torch.round(x.detach() / sa), -127, 127).reshape(-1, 64)
    wq = torch.clamp(torch.round(w / s[:, None]), -127, 127)
    assert torch.allclose(y.reshape(-1, 48), (xq @ wq.t()) * (sa * s)[None, :], atol=1e-6)
    dy = torch.randn(y.shape, generator=g)
    y.backward(dy)
    assert torch.allclose(x.grad.reshape(-1, 64), dy.reshape(-1, 48) @ (wq * s[:, None]), atol=1e-6)
    G = dy.reshape(-1, 48).t() @ (xq * sa)
    t = w / s[:, None]
    inside = (t.abs() <= 127) if method == "lsq" else torch.ones_like(t, dtype=torch.bool)
    assert torch.allclose(m.weight.grad, G * inside, atol=1e-4)
    if method == "lsq":
        term = torch.where(inside, torch.round(t) - t, torch.sign(t) * 127)
        assert torch.allclose(m.weight_scale.grad, (G * term).sum(1) / math.sqrt(64 * 127), atol=1e-5)
    else:
        assert not hasattr(m, "weight_scale")


def test_clipped_weights_get_no_gradient_and_push_the_step():
    m, g = _layer("lsq")
    with torch.no_grad():
        m.weight_scale.mul_(0.01)  # far too small a step: most weights clip
    x = torch.randn(16, 64, generator=g)
    m(x).sum().backward()
    t = m.weight.detach() / m.weight_scale.detach()[:, None]
    assert (t.abs() > 127).any()
    assert (m.weight.grad[t.abs() > 127] == 0).all()


def test_inactive_layer_is_bitwise_a_plain_linear():
    m, g = _layer("lsq")
    plain = Linear(64, 48)
    with torch.no_grad():
        plain.weight.copy_(m.weight)
    x = torch.randn(5, 64, generator=g)
    assert set_qat_active(m, False) == 1
    assert torch.equal(m(x), plain(x))
    set_qat_active(m, True)
    assert not torch.equal(m(x), plain(x))


def test_scale_init_and_refresh_follow_the_weights():
    m, _ = _layer("lsq")
    want = (m.weight.detach().abs().mean(1) * (2.0 / math.sqrt(127))).clamp_min(1e-6)
    assert torch.allclose(m.weight_scale.detach(), want, rtol=1e-6)
    with torch.no_grad():
        m.weight.mul_(3.0)
    assert refresh_lsq_weight_scales(m) == 1
    assert torch.allclose(m.weight_scale.detach(), 3.0 * want, rtol=1e-6)


def test_model_build_respects_exemption_and_init_sets_scales():
    from open_transformers_b200.config import load_config
    from open_transformers_b200.models import build_model, init_weights

    cfg = load_config("tiny_cpu", ["++model.qat.enabled=true", "++model.qat.exempt_first_n_blocks=1", "model.n_layers=2"])
    model = build_model(cfg.model)
    init_weights(model, 0)
    assert not isinstance(model.blocks[0].attn.wq, QuantLinear) and isinstance(model.blocks[1].attn.wq, QuantLinear)
    assert isinstance(model.blocks[1].ffn.w_down, QuantLinear) and not isinstance(model.embedding.output, QuantLinear)
    s = model.blocks[1].attn.wo.weight_scale.detach()
    assert (s > 0).all() and torch.allclose(s, model.blocks[1].attn.wo.lsq_optimal_scale(model.blocks[1].attn.wo.weight.detach()))
    names = [n for n, _ in model.named_parameters()]
    assert "blocks.1.attn.wq.weight_scale" in names and "blocks.0.attn.wq.weight_scale" not in names


def test_qat_run_trains_and_replays(tmp_path):
    """warm start for one step, then int8 with a step-size refresh every step; the audit replay reproduces the hash"""
    from open_transformers_b200.cli.audit_replay import audit_replay
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["++model.qat.enabled=true", "++model.qat.enable_at_step=1", "++model.qat.scale_refresh_every_n_steps=1",
                         "train.ckpt_every_steps=2"])
    res = train(cfg, device="cpu", data_root=tmp)
    assert len(res["hashes"]) == 3 and all(math.isfinite(l) for l in res["losses"])
    r = audit_replay(from_init=True, descriptor_checkpoint=res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3)
    assert r["match"] is True and r["state_hash"] == res["hashes"][-1][1]
    plain = train(tiny_cfg(tmp + "/p", []), device="cpu", data_root=tmp + "/p")
    assert plain["hashes"][-1][1] != res["hashes"][-1][1]


def test_block_hadamard_is_the_sign_matrix_and_cancels_in_a_product():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 256, generator=g)
    n = torch.arange(128)
    H = torch.tensor([[(-1.0) ** bin(int(i & j)).count("1") for j in n] for i in n])
    want = torch.cat([x[:, :128] @ H, x[:, 128:] @ H], 1)
    got = K.fwht_blocks(x)
    assert torch.allclose(got, want, atol=1e-4)
    assert torch.equal(got, K.fwht_blocks(x.clone()))
    y = torch.randn(7, 256, generator=g)
    assert torch.allclose(K.fwht_blocks(x) @ K.fwht_blocks(y).t() / 128, x @ y.t(), atol=1e-3)


def test_hadamard_int8_product_is_close_and_robust_to_an_outlier():
    g = torch.Generator().manual_seed(4)
    a, b = torch.randn(128, 256, generator=g), torch.randn(64, 256, generator=g)
    a[3, 17] = 200.0  # one outlier would cost a plainly quantised row almost all of its grid
    want = a @ b.t()
    got = K.ste_matmul_hadamard(a, b)
    assert got.dtype == torch.float32 and got.shape == (128, 64)
    assert (got - want).norm() / want.norm() < 0.02
    # the same rows quantised without the rotation: the outlier row is far worse
    aq, sa = K.quant_rows(a, 127)
    bq, sb = K.quant_rows(b, 127)
    plain = (aq.float() * sa[:, None]) @ (bq.float() * sb[:, None]).t()
    assert (got[3] - want[3]).norm() < 0.5 * (plain[3] - want[3]).norm()


@pytest.mark.parametrize("method", ["lsq", "absmax"])
def test_hadamard_backward_is_close_to_the_float_backward(method):
    def run(flag):
        g = torch.Generator().manual_seed(5)
        m = QuantLinear(128, 256, method=method, ste_bwd_hadamard=flag)
        with torch.no_grad():
            m.weight.copy_(torch.randn(256, 128, generator=g) * 0.05)
            if method == "lsq":
                m.weight_scale.copy_(m.lsq_optimal_scale(m.weight))
        x = torch.randn(2, 64, 128, generator=g, requires_grad=True)
        y = m(x)
        y.backward(torch.randn(y.shape, generator=g))
        return y.detach(), x.grad, m.weight.grad, (m.weight_scale.grad if method == "lsq" else None)

    y0, dx0, dw0, ds0 = run(False)
    y1, dx1, dw1, ds1 = run(True)
    assert torch.equal(y0, y1)  # the forward is untouched
    assert not torch.equal(dx0, dx1)
    assert (dx1 - dx0).norm() / dx0.norm() < 0.03 and (dw1 - dw0).norm() / dw0.norm() < 0.03
    if ds0 is not None:
        assert (ds1 - ds0).norm() / ds0.norm() < 0.1
    again = run(True)
    assert torch.equal(dx1, again[1]) and torch.equal(dw1, again[2])
    # a contraction length off the block falls back to the float GEMMs, bit for bit
    g = torch.Generator().manual_seed(6)
    x = torch.randn(3, 128, generator=g)
    outs = []
    for flag in (False, True):
        m, _ = _layer(method, 128, 256)
        m.ste_bwd_hadamard = flag
        xx = x.clone().requires_grad_(True)
        m(xx).sum().backward()
        outs.append((xx.grad, m.weight.grad))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_hadamard_qat_run_trains_and_replays(tmp_path):
    from open_transformers_b200.cli.audit_replay import audit_replay
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    over = ["++model.qat.enabled=true", "train.ckpt_every_steps=2"]
    res = train(tiny_cfg(tmp, over + ["++model.qat.ste_bwd_hadamard=true"]), device="cpu", data_root=tmp)
    assert all(math.isfinite(l) for l in res["losses"])
    r = audit_replay(from_init=True, descriptor_checkpoint=res["run_dir"] + "/checkpoints/step_000000002", data_root=tmp, until_step=3)
    assert r["match"] is True and r["state_hash"] == res["hashes"][-1][1]
    plain = train(tiny_cfg(tmp + "/p", over), device="cpu", data_root=tmp + "/p")
    assert plain["hashes"][-1][1] != res["hashes"][-1][1]  # the tiny model's shapes reach the int8 backward
    assert plain["losses"][0] == res["losses"][0]


# ------------------------------------------------------------------------------------------ GPU
def _both(fn, *cpu_args):
    a = fn(*cpu_args)
    b = fn(*[t.cuda() if isinstance(t, torch.Tensor) else t for t in cpu_args])
    return a, b


def _eq(a, b, what):
    a = a if isinstance(a, (tuple, list)) else (a,)
    b = b if isinstance(b, (tuple, list)) else (b,)
    for i, (x, y) in enumerate(zip(a, b)):
        if x is None:
            continue
        assert torch.equal(x, y.cpu()), "%s output %d differs: %d elements" % (what, i, int((x != y.cpu()).sum()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gpu_quant_kernels_bitwise(dtype):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(300, 328, generator=g) * 3).to(dtype)
    _eq(*_both(lambda t: K.quant_act(t, 127), x), "quant_act")
    w = (torch.randn(136, 328, generator=g) * 0.05).to(dtype)
    s = K.row_stat(w, "mean_abs", 2.0 / math.sqrt(127), 1e-6)
    _eq(*_both(lambda t: K.row_stat(t, "mean_abs", 2.0 / math.sqrt(127), 1e-6), w), "row_stat mean")
    _eq(*_both(lambda t: K.row_stat(t, "absmax", 1.0 / 127, 1e-12), w), "row_stat absmax")
    _eq(*_both(lambda t, u: K.quant_weight(t, u, 127, dtype), w, s), "quant_weight")
    _eq(*_both(lambda t, u: K.quant_weight(t, u * 0.02, 127, dtype), w, s), "quant_weight clipped")
    G = torch.randn(136, 328, generator=g)
    ga = torch.tensor([0.013])

    def bwd(G_, w_, s_, ga_):
        dW = torch.full_like(G_, 0.5)
        ds = torch.full_like(s_, 0.25)
        K.lsq_bwd_(G_, w_, s_ * 0.3, ga_, 127, 1.0 / math.sqrt(328 * 127), dW, ds)
        return dW, ds

    _eq(*_both(bwd, G, w, s, ga), "lsq_bwd")
    q = torch.randint(-127, 128, (1000,), generator=g, dtype=torch.int8)
    _eq(*_both(lambda t: K.i8_widen(t, dtype), q), "i8_widen")


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,Kd", [(200, 136, 336), (384, 512, 1024), (130, 96, 64)])
def test_gpu_int8_gemm_is_exact(M, N, Kd):
    """tcgen05 kind::i8 accumulates in int32, so the GPU result equals the integer sum on the host."""
    g = torch.Generator().manual_seed(4)
    a = torch.randint(-127, 128, (M, Kd), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (N, Kd), generator=g, dtype=torch.int8)
    sa = torch.tensor([0.0123])
    sb = torch.rand(N, generator=g) * 0.01 + 1e-3
    for dt in (torch.float32, torch.bfloat16):
        _eq(*_both(lambda a_, b_, sa_, sb_: K.gemm_i8(a_, b_, sa_, sb_, dt), a, b, sa, sb), "gemm_i8 %s" % dt)
    R = torch.randn(M, N, generator=g).bfloat16()
    _eq(*_both(lambda a_, b_, sa_, sb_, r_: K.gemm_i8(a_, b_, sa_, sb_, torch.bfloat16, r_), a, b, sa, sb, R), "gemm_i8 residual")
    exact = (a.double() @ b.double().t())
    got = K.gemm_i8(a.cuda(), b.cuda(), torch.ones(1).cuda(), torch.ones(N).cuda(), torch.float32).cpu().double()
    assert (got - exact).abs().max() <= exact.abs().max() * 2 ** -24
    assert K.kernel_status("cuda") == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mixed", [False, True])
def test_gpu_qat_engine_matches_cpu_hashes(mixed):
    from open_transformers_b200.config import load_config
    from open_transformers_b200.train.engine import TrainEngine

    extra = ["++model.qat.enabled=true", "++model.qat.scale_refresh_every_n_steps=2", "++model.qat.exempt_first_n_blocks=1"]
    if mixed:
        cfg = load_config("open1b_b200", ["model.n_layers=2", "model.d_model=256", "model.n_heads=2", "model.n_kv_heads=1", "model.ffn_intermediate=512",
                                          "model.vocab_size=1024", "train.seq_len=128", "data.seq_len=128", "run.virtual_dp_size=2", "run.dp_shard_size=2", *extra])
    else:
        cfg = load_config("tiny_cpu", extra)

    def run(device):
        eng = TrainEngine(cfg, device)
        g = torch.Generator().manual_seed(0)
        prev, out = None, []
        for _ in range(2):
            eng.zero_grads()
            for v in range(2):
                ids = torch.randint(0, 1024, (2, 128), generator=g).to(device)
                lab = torch.randint(0, 1024, (2, 128), generator=g).to(device)
                ce, _ = eng.forward_backward(v, ids, lab, 1)
            norm = eng.reduce_gradients()
            eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
            prev = eng.sharded_state_hash(prev, None, tensor_digest="tree")
            out.append((float(ce), norm, prev))
        return out

    cpu, gpu = run("cpu"), run("cuda")
    assert [h for _, _, h in cpu] == [h for _, _, h in gpu], (cpu, gpu)


# ------------------------------------------------------------------------------ int8 P V attention
def _attn_inputs(T=300, H=4, Hkv=2, D=128, seed=12):
    g = torch.Generator().manual_seed(seed)
    qk = torch.randn(T, (H + Hkv) * D, generator=g).bfloat16()
    qkv = torch.randn(T, (H + 2 * Hkv) * D, generator=g).bfloat16()
    return qk, qkv


@pytest.mark.parametrize("window", [0, 160])
def test_int8_pv_attention_is_close_to_the_float_kernel(window):
    qk, qkv = _attn_inputs()
    O0, l0 = K.attn_fwd(qk, qkv, 1, 300, 4, 2, 128, window)
    O1, l1 = K.attn_fwd(qk, qkv, 1, 300, 4, 2, 128, window, int8_pv=True)
    assert torch.equal(l0, l1)  # softmax statistics stay fp32 on the unquantised probabilities
    err = (O0.float() - O1.float()).abs().max().item()
    assert 0 < err < 0.05 * O0.float().abs().max().item()
    with pytest.raises(ValueError):
        K.attn_fwd(qk.float(), qkv.float(), 1, 300, 4, 2, 128, window, int8_pv=True)


def test_int8_pv_module_trains_with_the_float_shadow_backward():
    from open_transformers_b200.models.modules.core import GQAQKNorm
    from open_transformers_b200.ops import functional as KK

    torch.manual_seed(0)
    m = GQAQKNorm(256, 2, 1, 128, attn_int8_pv=True, qk_norm_gain=False).to(torch.bfloat16)
    ref = GQAQKNorm(256, 2, 1, 128, attn_int8_pv=False, qk_norm_gain=False).to(torch.bfloat16)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn_like(p.float()).mul(0.05))
    ref.load_state_dict(m.state_dict())
    cos, sin = KK.rope_tables(128, 128, 10000.0, "cpu")
    x = torch.randn(1, 128, 256).bfloat16().requires_grad_(True)
    y = m(x, cos, sin)
    y.float().square().sum().backward()
    y0 = ref(x.detach(), cos, sin)
    assert not torch.equal(y, y0) and (y.float() - y0.float()).abs().max() < 0.05 * y0.float().abs().max() + 1e-3
    assert torch.isfinite(x.grad.float()).all() and x.grad.float().abs().sum() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("window,T", [(0, 300), (160, 512)])
def test_gpu_int8_pv_attention_bitwise_vs_twin(window, T):
    qk, qkv = _attn_inputs(T=2 * T)
    cpu = K.attn_fwd(qk, qkv, 2, T, 4, 2, 128, window, int8_pv=True)
    gpu = K.attn_fwd(qk.cuda(), qkv.cuda(), 2, T, 4, 2, 128, window, int8_pv=True)
    _eq(cpu, gpu, "int8 P V attention")
    assert K.kernel_status("cuda") == 0


def test_every_recipe_switch_together_trains_and_replays_in_bf16(tmp_path):
    """bf16 compute, sliding-window layers, int8 P V, QK-norm gains, quantisation-aware layers past an exempt block with a
    step-size refresh, activation checkpointing: the run's digests are reproduced from its checkpoint and from the seed
    (the second time with folded gradients and offloaded moments)"""
    from open_transformers_b200.cli.audit_replay import audit_replay
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    over = ["run.mixed_precision=true", "model.n_layers=2", "model.swa_window=32", "model.swa_full_every=2", "model.attn_int8_pv=true", "model.head_dim=64",
            "model.n_heads=2", "model.n_kv_heads=1", "model.d_model=128", "train.seq_len=128", "data.seq_len=128", "model.max_seq_len_pretrain=128",
            "train.global_batch_tokens.warmup=512", "train.global_batch_tokens.main=512", "train.global_batch_tokens.late=512", "train.total_tokens=1536",
            "++model.qat.enabled=true", "++model.qat.exempt_first_n_blocks=1", "++model.qat.scale_refresh_every_n_steps=2", "train.ckpt_every_steps=2",
            "model.modules.attention=gqa_qknorm_repop", "model.qk_norm=true", "model.qk_norm_gain=true", "run.activation_checkpoint=true"]
    res = train(tiny_cfg(tmp, over), device="cpu", data_root=tmp)
    assert len({h for _, h in res["hashes"]}) == 3 and all(math.isfinite(l) for l in res["losses"])
    ck = res["run_dir"] + "/checkpoints/step_000000002"
    assert audit_replay(ck, data_root=tmp, until_step=3)["match"] is True
    r = audit_replay(from_init=True, descriptor_checkpoint=ck, data_root=tmp, until_step=3, offload_grads=True, offload_optimizer=True)
    assert r["match"] is True and r["state_hash"] == res["hashes"][-1][1]
