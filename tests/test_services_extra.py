"""Smaller services around the training loop: the stand-alone z-loss, QK-gain control, global-norm clip, the audit's
environment allow-list, CPU thread selection, the step -> document map, the interval fetcher and Muon.
(reference test strategy: tests/test_z_loss.py, tests/test_global_clip.py, tests/test_doc_map.py,
tests/test_fetch_interval.py, tests/test_cpu_threads.py)"""
import json
import math
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import tiny_cfg


# ------------------------------------------------------------------------------------------ z-loss
def test_z_loss_value_gradient_and_row_independence():
    from open_transformers_b200.models.fused_loss import fused_ce_z_loss
    from open_transformers_b200.models.z_loss import compute_z_loss, row_lse, z_loss_grad

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(6, 40, generator=g) * 3
    lse = row_lse(logits)
    assert torch.allclose(lse, torch.logsumexp(logits, -1), atol=1e-5)
    assert torch.equal(row_lse(logits[2:5]), lse[2:5])  # a row does not depend on its neighbours
    x = logits.clone().requires_grad_(True)
    z = compute_z_loss(x, 1e-2)
    z.backward()
    y = logits.clone().requires_grad_(True)
    zr = 1e-2 * torch.logsumexp(y, -1).square().mean()
    zr.backward()
    assert abs(float(z) - float(zr)) < 1e-6 and torch.allclose(x.grad, y.grad, atol=1e-6)
    assert torch.equal(z_loss_grad(logits, 1e-2, 1.0, chunk_rows=2), z_loss_grad(logits, 1e-2, 1.0, chunk_rows=6))
    # same bits as the z term of the fused loss
    _, zf = fused_ce_z_loss(logits.clone(), torch.zeros(6, dtype=torch.long), 1e-2)
    assert float(zf) == float(z)

    class Off:
        enabled, coeff = False, 1e-2

    assert float(compute_z_loss(logits, Off())) == 0.0 and not compute_z_loss(x, 0.0).requires_grad


# ------------------------------------------------------------------------------------- QK-gain control
def test_qk_gain_clamp_and_frozen_query_gains():
    from open_transformers_b200.models.modules.core import GQAQKNorm
    from open_transformers_b200.train.qk_gain_control import clamp_qk_gains, zero_q_gain_grads

    m = GQAQKNorm(64, 2, 1, 32)
    with torch.no_grad():
        m.q_norm.weight.fill_(3.0)
        m.k_norm.weight.fill_(0.5)
    assert clamp_qk_gains(m, 0.0) == 0 and float(m.q_norm.weight[0]) == 3.0
    assert clamp_qk_gains(m, 2.0) == 2
    assert float(m.q_norm.weight.max()) == 2.0 and float(m.k_norm.weight.max()) == 0.5
    with torch.no_grad():
        m.k_norm.weight[3] = -7.0  # the clamp is symmetric: a gain drifting below -cap is bounded too
    clamp_qk_gains(m, 2.0)
    assert float(m.k_norm.weight.min()) == -2.0
    grads = {"attn.q_norm.weight": torch.ones(32), "attn.k_norm.weight": torch.ones(32), "attn.wq.weight": torch.ones(4, 4)}
    assert zero_q_gain_grads(grads, step=3, freeze_until_step=5) == 1
    assert float(grads["attn.q_norm.weight"].sum()) == 0.0 and float(grads["attn.k_norm.weight"].sum()) == 32.0
    assert zero_q_gain_grads(grads, step=5, freeze_until_step=5) == 0


# ---------------------------------------------------------------------------------------- global clip
def test_global_norm_and_clip():
    from open_transformers_b200.train.global_clip import clip_coefficient, clip_grads_, deterministic_global_norm

    g = torch.Generator().manual_seed(1)
    named = [("a", torch.randn(32, 8, generator=g)), ("b", torch.randn(8, generator=g)), ("c", None), ("d", torch.randn(64, 64, generator=g))]
    norm, per = deterministic_global_norm(named, num_shards=2)
    ref = math.sqrt(sum(float(t.double().square().sum()) for _, t in named if t is not None))
    assert abs(norm - ref) < 1e-4 * ref and len(per) == 3
    assert deterministic_global_norm(named, 2)[0] == norm  # same call, same bits
    assert clip_coefficient(norm, 0.0) == 1.0 and clip_coefficient(0.5, 1.0) == 1.0
    assert abs(clip_coefficient(4.0, 1.0) - 0.25) < 1e-6
    pre = clip_grads_(named, 1.0, 2)
    assert pre == norm
    post, _ = deterministic_global_norm(named, 2)
    assert abs(post - 1.0) < 1e-3


# ------------------------------------------------------------------------------ audit environment allow-list
def test_audit_env_allow_list(monkeypatch):
    from open_transformers_b200.cli.audit_replay import AuditError, apply_kernel_env

    monkeypatch.delenv("OTB_TENSOR_DIGEST", raising=False)
    applied = apply_kernel_env({"OTB_TENSOR_DIGEST": "tree", "SOME_OTHER_KEY": "x"})
    assert applied == {"OTB_TENSOR_DIGEST": "tree"} and os.environ["OTB_TENSOR_DIGEST"] == "tree" and "SOME_OTHER_KEY" not in os.environ
    for bad in ("LD_PRELOAD", "PYTHONPATH", "OTB_LIB_DIR", "OTB_CXX"):
        with pytest.raises(AuditError):
            apply_kernel_env({bad: "/tmp/evil"})


# ----------------------------------------------------------------------------------------- cpu threads
def test_cpu_threads_parsing():
    from open_transformers_b200.cli.cpu_threads import available_cpus, configure_cpu_threads, parse_cpu_threads

    assert parse_cpu_threads("auto") == available_cpus() >= 1 and parse_cpu_threads(None) == available_cpus()
    assert parse_cpu_threads("3") == 3 and parse_cpu_threads(2) == 2
    for bad in ("0", -1):
        with pytest.raises(ValueError):
            parse_cpu_threads(bad)
    before = torch.get_num_threads()
    assert configure_cpu_threads(1) == 1 and os.environ["OMP_NUM_THREADS"] == "1"
    configure_cpu_threads(before)


# ------------------------------------------------------------------------- doc map and interval fetcher
def test_doc_map_covers_every_window_slot_and_fetch_interval_brings_only_touched_shards(tmp_path):
    import pandas as pd
    import pyarrow.parquet as pq

    from open_transformers_b200.data.doc_map import COLUMNS, compare_position, write_doc_map
    from open_transformers_b200.data.fetch_interval import DirMirror, fetch_audit_interval
    from open_transformers_b200.data.loader import build_global_loader
    from open_transformers_b200.train.loop import train

    tmp = str(tmp_path)
    cfg = tiny_cfg(tmp, ["train.ckpt_every_steps=1"])
    V = cfg.run.virtual_dp_size or 2
    view = build_global_loader(cfg, [], 1, data_root=tmp, index_only=True)
    out = tmp_path / "doc_map"
    summary = write_doc_map(view, out, until_step=2, micro_batch_size=cfg.train.micro_batch_size, dp_world_size=V, chunk_steps=1)
    assert [Path(f).name for f in summary["files"]] == ["step_docs-000000-000000.parquet", "step_docs-000001-000001.parquet"]
    tab = pd.concat([pq.read_table(f).to_pandas() for f in summary["files"]])
    assert tuple(tab.columns) == COLUMNS and len(tab) == summary["rows"] > 0 and summary["steps_walked"] == 2
    per_step = cfg.train.global_batch_tokens.warmup // cfg.train.seq_len
    assert set(tab["step"]) == {0, 1} and summary["windows"] == 2 * per_step
    # every window slot of every micro-batch is covered by document pieces that add up to seq_len + 1 tokens or less; the
    # pieces of a window are numbered from 0, and the global window index follows (step, micro-batch, slot)
    tab["length"] = tab["tok_end"] - tab["tok_start"]
    grp = tab.groupby(["step", "microbatch", "slot"])["length"].sum()
    assert len(grp) == 2 * per_step and int(grp.max()) <= cfg.train.seq_len + 1 and int(grp.min()) > 0
    assert set(tab["dp_rank"]) <= set(range(V)) and tab.groupby("global_window")["frag_idx"].min().eq(0).all()
    mb = cfg.train.micro_batch_size
    assert ((tab["global_window"] - tab["step"] * per_step) == tab["microbatch"] * mb + tab["slot"]).all()
    assert sum(summary["rows_per_source"].values()) == summary["rows"]
    # the position a walk ends at is what a training run records after the same steps
    assert summary["position"]["windows_emitted"] == 2 * per_step

    res = train(cfg, device="cpu", data_root=tmp, max_steps=2)
    ck = Path(res["run_dir"]) / "checkpoints" / "step_000000001"
    recorded = json.loads((Path(res["run_dir"]) / "checkpoints" / "step_000000002" / "global_stream.json").read_text())
    assert compare_position(summary["position"], recorded) == []
    assert compare_position(dict(summary["position"], windows_emitted=1), recorded) == ["windows_emitted: walk=1 ckpt=%d" % (2 * per_step)]
    dest = tmp_path / "fetched"
    fetch_audit_interval(ck, DirMirror(tmp), dest, until_step=2)
    from open_transformers_b200.cli.audit_replay import audit_replay

    r = audit_replay(str(ck), data_root=str(dest), until_step=2, expect_hash=res["hashes"][-1][1])
    assert r["match"] is True


# ------------------------------------------------------------------------------------------------ Muon
def test_muon_orthogonalises_and_the_aux_optimizer_takes_the_rest():
    from open_transformers_b200.optim.muon import Muon, MuonWithAuxAdamW, newton_schulz5

    g = torch.Generator().manual_seed(2)
    G = torch.randn(32, 16, generator=g)
    O = newton_schulz5(G)
    sv = torch.linalg.svdvals(O)
    assert float(sv.max()) < 1.3 and float(sv.min()) > 0.3  # singular values pushed toward one
    w = torch.nn.Parameter(torch.randn(8, 8, generator=g))
    b = torch.nn.Parameter(torch.zeros(8))
    from open_transformers_b200.config.schema import OptimConfig

    opt = MuonWithAuxAdamW([("blocks.0.w", w), ("blocks.0.b", b)], OptimConfig(), muon_lr=0.02)
    (w.sum() + b.sum()).backward()
    before = w.detach().clone()
    opt.step()
    opt.zero_grad()
    assert not torch.equal(before, w.detach()) and float(b.detach().abs().sum()) > 0
    assert isinstance(opt.muon, Muon)


def test_muon_hybrid_in_the_engine_updates_hidden_matrices_orthogonally_and_the_rest_by_adamw(tmp_path):
    import numpy as np

    from open_transformers_b200.config import load_config
    from open_transformers_b200.train.engine import TrainEngine

    def run(name, steps=2):
        cfg = load_config("tiny_cpu", ["optim.name=%s" % name])
        eng = TrainEngine(cfg, "cpu")
        before = {n: p.clone() for n, p in eng.named_master()}
        g = torch.Generator().manual_seed(0)
        for _ in range(steps):
            eng.zero_grads()
            for v in range(eng.V):
                ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
                eng.forward_backward(v, ids, torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), 1)
            norm = eng.reduce_gradients()
            eng.optimizer_step(1e-2, eng.clip_coefficient(norm, 1.0))
        after = dict(eng.named_master())
        return eng, before, after

    eng, before, after = run("muon_hybrid")
    hidden = [eng.names[i] for i in eng.muon_params]
    assert hidden and all("embedding" not in n and "norm" not in n for n in hidden)
    assert any(n.endswith("wo.weight") for n in hidden) and any("w_down" in n for n in hidden)
    _, b2, a2 = run("adamw")
    for n in before:
        assert not torch.equal(before[n], after[n]) or "norm" in n, n          # everything trains
    for n in hidden:   # Muon's step is (nearly) orthogonal: its singular values sit near 1, unlike AdamW's
        d = (after[n] - before[n] * (1 - 1e-2 * eng.cfg.optim.weight_decay) ** 2)
        assert not torch.equal(after[n], a2[n])
        sv = torch.linalg.svdvals(d.float())
        assert sv.max() / sv.median() < 4.0, (n, sv.max() / sv.median())
    emb = [n for n in before if "embedding" in n]
    _, _, m1 = run("muon_hybrid", 1)
    _, _, p1 = run("adamw", 1)
    assert emb and all(torch.equal(m1[n], p1[n]) for n in emb)                  # the aux AdamW is the engine's kernel
    assert float(eng.m2[eng.layout.offsets[eng.muon_params[0]]]) == 0.0
    eng.close()


def test_audit_memory_log_is_opt_in(monkeypatch):
    from open_transformers_b200.cli.audit_replay import memlog

    monkeypatch.delenv("PRETRAIN_AUDIT_MEMLOG", raising=False)
    assert memlog("x") is None
    monkeypatch.setenv("PRETRAIN_AUDIT_MEMLOG", "1")
    rec = memlog("after load")
    assert rec["at"] == "after load" and rec["rss_peak_gib"] > 0 and rec.get("rss_gib", 1) > 0 and "cuda_peak_gib" not in rec


def test_replay_memory_plan_switches_offloads_on_in_order_and_keeps_requests():
    from open_transformers_b200.cli.audit_replay import memory_plan
    from open_transformers_b200.config import load_config
    from open_transformers_b200.models import build_model
    from open_transformers_b200.obs.metrics import count_parameters

    for name in ("tiny_cpu", "100m_smoke_repop"):
        cfg = load_config(name)
        with torch.device("meta"):
            model = build_model(cfg.model)
        lsq = sum(p.numel() for n, p in model.named_parameters() if n.endswith("weight_scale"))
        assert count_parameters(cfg.model) == model.num_parameters() - lsq, name
    n, G = 1_600_000_000, 2 ** 30
    act, reserve = 24 * G, 4 * G
    roomy = memory_plan(n, 8, 1, True, act, 180 * G, reserve, False, False)
    assert roomy["auto"] == [] and roomy["fits"] and not roomy["offload_grads"]
    assert abs(roomy["need_bytes"] - (n * (18 + 32) + act + reserve)) == 0
    tight = memory_plan(n, 8, 1, True, act, 80 * G, reserve, False, False)           # 102.5 GiB by default: fold the gradients
    assert tight["auto"] == ["offload_grads"] and tight["fits"] and not tight["offload_optimizer"]
    tighter = memory_plan(n, 8, 1, True, act, 60 * G, reserve, False, False)         # 66.7 GiB folded: moments go too
    assert tighter["auto"] == ["offload_grads", "offload_optimizer"] and tighter["fits"]
    hopeless = memory_plan(n, 8, 1, True, act, 20 * G, reserve, False, False)
    assert not hopeless["fits"] and hopeless["offload_optimizer"] and hopeless["offload_grads"]
    asked = memory_plan(n, 8, 1, True, act, 180 * G, reserve, True, True)
    assert asked["auto"] == [] and asked["offload_grads"] and asked["offload_optimizer"]
    assert memory_plan(n, 8, 1, True, act, None, reserve, False, False)["auto"] == []
    assert memory_plan(n, 2, 1, True, act, 40 * G, reserve, False, False)["auto"] == ["offload_optimizer"]  # folding 2 -> 2 buffers gains nothing


def test_standalone_adamw_and_clip_helpers_give_the_engine_bits():
    """the torch.optim-style AdamW and the plain-tensor norm / clip helpers against the flat-buffer engine, on the same
    gradients: identical norm, identical updated weights and moments, two steps (bias corrections advance)"""
    from torch import nn

    from open_transformers_b200.config import load_config
    from open_transformers_b200.optim.adamw import build_adamw, prime_optimizer_state
    from open_transformers_b200.optim.registry import build_optimizer
    from open_transformers_b200.train.engine import TrainEngine
    from open_transformers_b200.train.global_clip import clip_coefficient, deterministic_global_norm

    cfg = load_config("tiny_cpu")
    eng = TrainEngine(cfg, "cpu")
    params = [(n, nn.Parameter(p.detach().clone())) for n, p in eng.named_master()]
    opt = build_optimizer(params, cfg.optim)
    assert type(opt).__name__ == "DeterministicAdamW" and type(build_adamw(params, cfg.optim)) is type(opt)
    prime_optimizer_state(opt)
    assert all(int(opt.state[p]["step"]) == 0 for _, p in params)
    g = torch.Generator().manual_seed(0)
    for step in range(2):
        eng.zero_grads()
        for v in range(eng.V):
            ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
            eng.forward_backward(v, ids, torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), 1)
        norm = eng.reduce_gradients()
        grads = eng.named_grads()
        norm2, _ = deterministic_global_norm([(n, grads[n]) for n in eng.names], eng.dp_shard)
        assert norm2 == norm
        clip = eng.clip_coefficient(norm, 0.5)
        assert clip == clip_coefficient(norm, 0.5) and clip < 1.0
        for n, p in params:
            p.grad = grads[n].detach().clone()
        for group in opt.param_groups:
            group["lr"] = 1e-3
        opt.step(clip=clip)
        eng.optimizer_step(1e-3, clip)
        after = dict(eng.named_master())
        state = eng.optimizer_state()
        for n, p in params:
            assert torch.equal(p.detach(), after[n]), (step, n)
            assert torch.equal(opt.state[p]["exp_avg"], state[n]["exp_avg"]) and torch.equal(opt.state[p]["exp_avg_sq"], state[n]["exp_avg_sq"]), n
    eng.close()


def test_hardware_flops_count_the_causal_mask_the_window_and_grouped_projections():
    """8.54 GFLOP per token for the OPEN-1B shape (the reference's dense formula says 11.24): 6 per matrix weight, and per
    layer 12 d per visible (query, key) pair - (T + 1) / 2 keys under the causal mask, about 480 under the 512-key window."""
    from open_transformers_b200.config import load_config
    from open_transformers_b200.obs.metrics import hardware_flops_per_token, transformer_flops_per_token

    m = load_config("open1b_b200", []).model
    hw = hardware_flops_per_token(m, 4096)
    weights = 24 * (2048 * 2048 * 2 + 2048 * 512 * 2 + 3 * 2048 * 5632) + 128256 * 2048
    window_keys = (512 * 513 / 2 + (4096 - 512) * 512) / 4096
    assert hw == pytest.approx(6 * weights + 12 * 2048 * (5 * 2048.5 + 19 * window_keys))
    assert 8.5e9 < hw < 8.6e9 < transformer_flops_per_token(24, 2048, 4096, 128256)
    m2 = m.model_copy(update={"swa_window": 0})
    assert hardware_flops_per_token(m2, 4096) == pytest.approx(6 * weights + 12 * 2048 * 24 * 2048.5)


def test_compiled_distribution_hook_translates_a_module_and_keeps_its_behaviour(tmp_path):
    """setup.py's PRETRAIN_PYTHON_NATIVE path on one module: Cython translates `optim/schedules.py`, the C file is built
    with -ffp-contract=off, the extension imports in place of the source and computes the same learning rates; package
    markers stay source, and the recorded commit comes from PRETRAIN_BUILD_COMMIT when it is set."""
    import importlib.util
    import os
    import shutil
    import subprocess
    import sys
    import sysconfig
    from pathlib import Path

    pytest.importorskip("Cython")
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("otb_setup", root / "setup.py")
    hook = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(hook)
    mods = hook.compiled_modules()
    assert len(mods) > 40 and not any(p.name in ("__init__.py", "__main__.py", "build_native.py") for p in mods)
    os.environ["PRETRAIN_BUILD_COMMIT"] = "abc123"
    try:
        assert hook.build_commit() == "abc123"
    finally:
        del os.environ["PRETRAIN_BUILD_COMMIT"]
    work = tmp_path / "w"
    (work / "pkg").mkdir(parents=True)
    shutil.copy(root / "open_transformers_b200" / "optim" / "schedules.py", work / "pkg" / "schedules.py")
    (work / "pkg" / "__init__.py").write_text("")
    exts = hook.cython_extensions([work / "pkg" / "schedules.py"], root=work, build_dir=str(work / "c"))
    assert exts[0].name == "pkg.schedules" and "-ffp-contract=off" in exts[0].extra_compile_args
    c_file = Path(exts[0].sources[0])
    so = work / "pkg" / ("schedules" + sysconfig.get_config_var("EXT_SUFFIX"))
    cc = sysconfig.get_config_var("CC").split()[0]
    r = subprocess.run([cc, "-shared", "-fPIC", *exts[0].extra_compile_args, "-I", sysconfig.get_paths()["include"], str(c_file), "-o", str(so)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    (work / "pkg" / "schedules.py").unlink()                                   # only the extension is left
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r); import pkg.schedules as c; "
            "from open_transformers_b200.optim import schedules as s; "
            "from open_transformers_b200.config import load_config; cfg = load_config('tiny_cpu', []); "
            "a = c.build_schedule(cfg.schedule, cfg.train, cfg.optim); b = s.build_schedule(cfg.schedule, cfg.train, cfg.optim); "
            "assert c.__file__.endswith('.so'); assert [a(t, 768) for t in range(0, 768, 64)] == [b(t, 768) for t in range(0, 768, 64)]; print('same')"
            % (str(work), str(root)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "same" in r.stdout, r.stderr[-2000:]


def test_amsgrad_variant_of_the_adamw_kernel_follows_torch():
    """the kernel's optional running maximum of the second moment against torch.optim.AdamW(amsgrad=True): a gradient that
    shrinks after the first steps keeps dividing by the early, larger second moment"""
    from open_transformers_b200.optim.adamw import DeterministicAdamW

    g = torch.Generator().manual_seed(5)
    w0 = torch.randn(3, 10_000, generator=g)
    grads = [torch.randn(3, 10_000, generator=g) * s for s in (1.0, 2.0, 0.1, 0.05, 0.5)]
    ours, ref = torch.nn.Parameter(w0.clone()), torch.nn.Parameter(w0.clone())
    a = DeterministicAdamW([ours], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=True)
    b = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=True)
    plain = torch.nn.Parameter(w0.clone())
    c = DeterministicAdamW([plain], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for gr in grads:
        for p, o in ((ours, a), (ref, b), (plain, c)):
            p.grad = gr.clone()
            o.step()
    assert torch.allclose(ours, ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(a.state[ours]["max_exp_avg_sq"], b.state[ref]["max_exp_avg_sq"], rtol=1e-6, atol=1e-12)
    assert bool((a.state[ours]["max_exp_avg_sq"] >= a.state[ours]["exp_avg_sq"]).all()) and not torch.equal(ours, plain)
    assert "max_exp_avg_sq" not in c.state[plain]


def test_linear_forward_hands_the_first_use_after_an_update_to_the_gathering_gemm():
    """the hook of ``run.param_sharding: gather`` in the linear layer's forward: while the weight's descriptor reports rows
    still to pull, the forward goes through it (once); afterwards, and in the backward pass, the plain GEMM runs"""
    import torch

    from open_transformers_b200.ops import autograd as A
    from open_transformers_b200.ops import functional as K

    class FakeGather:
        def __init__(self, w):
            self.w, self.todo, self.calls = w, True, []

        def pending(self):
            return self.todo

        def gemm(self, x, residual=None):
            self.calls.append(residual is not None)
            self.todo = False
            return K.gemm(x, self.w, epi=K.EPI_RESIDUAL, residual=residual) if residual is not None else K.gemm(x, self.w)

    g = torch.Generator().manual_seed(0)
    w = torch.randn(48, 32, generator=g).requires_grad_()
    x = torch.randn(2, 8, 32, generator=g).requires_grad_()
    res = torch.randn(2, 8, 48, generator=g)
    slot = A.GradSlot(torch.zeros(48, 32))
    slot.fresh = True
    plain = A.linear(x, w, None, None, res)
    slot.gather = FakeGather(w.detach())
    first = A.linear(x, w, w.detach(), slot, res)
    second = A.linear(x, w, w.detach(), slot, res)
    assert slot.gather.calls == [True] and torch.equal(first, plain) and torch.equal(second, plain)
    first.sum().backward()
    assert torch.equal(slot.buf, torch.einsum("btn,btk->nk", torch.ones_like(res), x.detach())) or torch.allclose(
        slot.buf, torch.einsum("btn,btk->nk", torch.ones_like(res), x.detach()), atol=1e-5)


def test_host_threads_block_changes_the_thread_count_and_not_the_bytes():
    """start-up work on the host of a GPU run may use this process's share of the cores although the launcher pinned
    OMP_NUM_THREADS to 1: the count is restored afterwards and the Philox samples do not depend on it"""
    import torch

    from open_transformers_b200.ops import functional as K
    from open_transformers_b200.ops.native import cpu_lib, host_threads

    before = int(cpu_lib().otb_cpu_set_threads(0))
    a, b = torch.empty(300_001), torch.empty(300_001)
    with host_threads(1):
        K.trunc_normal_(a, 0.02, 7, 11)
    with host_threads(3) as ht:
        assert ht.n == 3 and int(cpu_lib().otb_cpu_set_threads(0)) == 3
        K.trunc_normal_(b, 0.02, 7, 11)
    assert torch.equal(a, b) and int(cpu_lib().otb_cpu_set_threads(0)) == before
    assert host_threads().n >= 1


def test_gather_mode_plan_splits_the_owned_chunks_and_describes_every_projection(monkeypatch):
    """the planning half of ``run.param_sharding: gather`` on a CPU stand-in for two GPUs: every projection weight (the fused
    QKV operand as three row-concatenated weights) gets a descriptor whose rows-per-owner match the ownership, and the
    owned chunks split exactly into those the AdamW kernel keeps local (pulled weights) and those it pushes (the rest)"""
    import torch

    from open_transformers_b200.config import load_config
    from open_transformers_b200.train.engine import TrainEngine

    cfg = load_config("tiny_cpu", ["model.n_layers=2", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2", "model.ffn_intermediate=256",
                                   "model.vocab_size=256", "train.seq_len=64", "data.seq_len=64", "model.max_seq_len_pretrain=64",
                                   "run.virtual_dp_size=4", "run.dp_shard_size=4", "run.dp_replicate_size=1", "run.mixed_precision=true"])
    eng = TrainEngine(cfg, "cpu", 0, 1)
    assert eng._pg is None                                               # one process: nothing to gather
    lay = eng.layout
    # dress the engine up as rank 0 of two GPU processes with peer memory
    eng.world, eng.is_cuda, eng.peer, eng.sharded = 2, True, True, True
    eng._owner_ranges = lay.owner_ranges(2)
    eng.seg_lo, eng.seg_hi = eng._owner_ranges[0]
    eng.chunk_lo, eng.chunk_hi = int(lay.seg_first[eng.seg_lo]), int(lay.seg_first[eng.seg_hi])
    eng.buf_compute.ptrs = [eng.compute.data_ptr(), eng.compute.data_ptr()]
    monkeypatch.setenv("OTB_PARAM_SHARDING", "gather")
    eng._setup_param_gather()
    pg = eng._pg
    names = {lay.names[i] for i in pg["pulled_params"]}
    assert {n for n in lay.names if n.endswith((".wq.weight", ".wk.weight", ".wv.weight", ".wo.weight", ".w_gate_up.weight", ".w_down.weight"))} <= names
    assert "embedding.output.weight" in names and not any("tok_embeddings" in n or "norm" in n for n in names)
    fused = [g for g in pg["weights"] if g._nseg == 3]
    assert len(fused) == cfg.model.n_layers and all(list(g._seg) == [0, 128, 256] and list(g._rpo) == [64, 64, 64] for g in fused)
    assert all(not g.pending() for g in pg["weights"])                   # start-up: every process holds the whole weights
    pull, push = pg["tables"]["pull"], pg["tables"]["push"]
    owned = sum(s.length for s in lay.segments[eng.seg_lo:eng.seg_hi])
    assert int(pull[1].sum()) + int(push[1].sum()) == owned and pull[4] + push[4] == eng.chunk_hi - eng.chunk_lo
    starts = torch.cat([pull[0], push[0]])
    assert starts.unique().numel() == starts.numel()                     # no chunk in both tables
    pulled_elems = sum(s.length for s in lay.segments[eng.seg_lo:eng.seg_hi] if s.param in set(pg["pulled_params"]))
    assert int(pull[1].sum()) == pulled_elems


def test_small_helpers_under_the_reference_names(tmp_path):
    """tokens_per_sec, tokens_per_optimizer_step, rank / world_size / is_main_process outside a process group, and
    compute_perplexity over a held-out shard."""
    import math
    from types import SimpleNamespace

    import numpy as np

    from open_transformers_b200.data.indexed_dataset import IndexedDatasetWriter
    from open_transformers_b200.eval.perplexity import compute_perplexity
    from open_transformers_b200.obs.metrics import tokens_per_sec
    from open_transformers_b200.parallel import env
    from open_transformers_b200.train.batch_schedule import grad_accum_steps, tokens_per_optimizer_step

    assert tokens_per_sec(1000, 0.5) == 2000.0 and tokens_per_sec(1, 0.0) > 9e8
    assert env.rank() == 0 and env.world_size() == 1 and env.is_main_process()
    from open_transformers_b200.config.schema import GlobalBatchTokens, TrainConfig

    train = TrainConfig(micro_batch_size=2, seq_len=16, global_batch_tokens=GlobalBatchTokens(warmup=200, main=512, late=1024),
                        warmup_to_main_at_tokens=1000, main_to_late_at_tokens=5000)
    assert grad_accum_steps(0, train, 2) == 4          # ceil(200 / (2 * 16 * 2))
    assert tokens_per_optimizer_step(0, train, dp_world_size=2) == 4 * 2 * 16 * 2
    assert tokens_per_optimizer_step(2000, train, dp_world_size=2) == 512 and tokens_per_optimizer_step(9000, train, dp_world_size=4) == 1024

    class Uniform(torch.nn.Module):
        def __init__(self, vocab):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(1))
            self.vocab = vocab

        def forward(self, ids):
            return SimpleNamespace(logits=torch.zeros(ids.shape + (self.vocab,), dtype=torch.float32) + self.w)

    with IndexedDatasetWriter(tmp_path / "held") as w:
        rng = np.random.default_rng(0)
        for n in (9, 17, 5):
            w.add_document(rng.integers(0, 64, n))
    ppl = compute_perplexity(Uniform(64), tmp_path / "held", seq_len=8, micro_batch_size=2)
    assert math.isclose(ppl, 64.0, rel_tol=1e-5)


def test_tensor_level_helpers_rope_zloss_norm():
    """apply_rope equals the fused QK-norm / RoPE kernel with the norm switched off; the inert z-loss has the value and no
    gradient; the total-norm helpers agree with the clip module; seeded init repeats."""
    from types import SimpleNamespace

    from open_transformers_b200.models.init import init_weights_seeded
    from open_transformers_b200.models.modules.core import apply_rope
    from open_transformers_b200.models.z_loss import compute_z_loss, compute_z_loss_inert
    from open_transformers_b200.ops import functional as K
    from open_transformers_b200.parallel import deterministic_reduce as DR
    from open_transformers_b200.train.global_clip import deterministic_global_norm
    from open_transformers_b200.train.loop import cross_entropy_loss

    g = torch.Generator().manual_seed(4)
    B, T, H, D = 2, 24, 3, 16
    x = torch.randn(B, T, H * D, generator=g)
    cos, sin = K.rope_tables(T, D, 10000.0, "cpu")
    fused = K.qknorm_rope_fwd(x.reshape(B * T, H * D).clone(), cos, sin, H, D, T, False, 1e-5)[0]
    assert torch.allclose(apply_rope(x.view(B, T, H, D), cos, sin).reshape(B, T, H * D), fused.reshape(B, T, H * D), atol=1e-6)

    logits = torch.randn(6, 32, generator=g, requires_grad=True)
    cfg = SimpleNamespace(enabled=True, coeff=1e-3)
    inert = compute_z_loss_inert(logits, cfg)
    assert not inert.requires_grad and torch.equal(inert, compute_z_loss(logits, cfg).detach())
    labels = torch.randint(0, 32, (6,), generator=g)
    assert torch.allclose(cross_entropy_loss(logits.detach(), labels), torch.nn.functional.cross_entropy(logits.detach(), labels), atol=1e-6)

    grads = [("a", torch.randn(33, 8, generator=g)), ("b", torch.randn(16, generator=g))]
    norm, per = deterministic_global_norm(grads, 2)
    assert DR.deterministic_total_norm(grads, 2) == norm == DR.audit_total_norm(grads, 2)
    assert DR.grad_sum_of_squares(grads, 2).tobytes() == per.tobytes()
    assert abs(norm - float(torch.cat([t.flatten() for _, t in grads]).norm())) < 1e-4

    m1, m2 = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)
    init_weights_seeded(m1, 5), init_weights_seeded(m2, 5)
    assert torch.equal(m1.weight, m2.weight) and float(m1.bias.detach().abs().sum()) == 0.0


def test_build_info_names_backends_and_commit():
    import open_transformers_b200 as pkg

    info = pkg.build_info()
    assert info["version"] == pkg.__version__ and "cpu" in info["backends"] and isinstance(info["native_source_digests"], dict)
    assert info["commit"] and isinstance(info["python_native"], bool)
