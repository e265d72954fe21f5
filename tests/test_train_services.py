import math
import pickle

import pytest
import torch

from open_transformers_b200.config import load_config
from open_transformers_b200.optim.schedules import build_schedule, rewarm_factor
from open_transformers_b200.train.checkpoint import (Checkpointer, UntrustedCheckpointError, validate_dcp_metadata)
from open_transformers_b200.train.midtrain import MidtrainConfigError, check_linear_anneal_resume
from open_transformers_b200.train.spike_protocol import Halt, SpikeProtocol
from open_transformers_b200.obs.metrics import mfu, transformer_flops_per_token


def test_schedules():
    cfg = load_config("1b_repop_v2")
    s = build_schedule(cfg.schedule, cfg.train, cfg.optim)
    warm = 667 * 3_145_728
    assert s(0) == 0.0 and s(warm) == pytest.approx(4.5e-4) and s(warm // 2) == pytest.approx(2.25e-4, rel=1e-6)
    assert s(cfg.train.total_tokens) == pytest.approx(4.5e-5)
    w = load_config("1b_repop_v2", ["schedule=wsd"])
    sw = build_schedule(w.schedule, w.train, w.optim)
    assert sw(int(0.5 * w.train.total_tokens)) == pytest.approx(4.5e-4) and sw(w.train.total_tokens) == pytest.approx(4.5e-5)
    m = load_config("1b_midtrain_math")
    sm = build_schedule(m.schedule, m.train, m.optim)
    assert sm(400_000_000_000) == pytest.approx(4.5e-5) and sm(405_000_000_000) == pytest.approx(2.25e-5) and sm(410_000_000_000) == 0.0
    assert rewarm_factor(150, 100, 100) == 0.5 and rewarm_factor(10, None, 100) == 1.0


def test_flops_formula():
    f = transformer_flops_per_token(24, 2048, 4096, 128256)
    assert f == pytest.approx(11.24e9, rel=2e-3)
    assert mfu(1000.0, f, 1e15) == pytest.approx(1000.0 * f / 1e15)


def test_spike_protocol_cooldown_halt_and_state():
    sp = SpikeProtocol(5.0, skips_in_window_to_halt=3, halt_window_steps=100, skip_steps_on_spike=3, start_step=10)
    assert not sp.should_skip(100.0, 1.0, step=5)            # before start_step
    assert sp.should_skip(1.0, float("nan"), step=5)          # non-finite loss always skips
    assert sp.should_skip(6.0, 1.0, step=10)
    sp.record_skip(10)
    assert sp.should_skip(0.1, 1.0, step=11)                  # cool-down
    sd = sp.state_dict()
    sp2 = SpikeProtocol(5.0, 3, 100, 3, 10)
    sp2.load_state_dict(sd)
    for s in (11, 12):
        assert sp2.should_skip(0.1, 1.0, step=s)
        sp2.record_skip(s)
    assert not sp2.should_skip(0.1, 1.0, step=13)
    sp2.record_skip(20)
    sp2.record_skip(21); sp2.record_skip(22)
    with pytest.raises(Halt):
        sp2.record_skip(30)
    assert sp2.state.halted and sp2.state.skipped_steps == 7


def test_midtrain_guards():
    cfg = load_config("1b_midtrain_math")
    check_linear_anneal_resume(cfg, 400_000_000_000)
    with pytest.raises(MidtrainConfigError):
        check_linear_anneal_resume(cfg, None)
    with pytest.raises(MidtrainConfigError):
        check_linear_anneal_resume(cfg, 399_000_000_000)
    cfg.train.resume_reset_optimizer = True
    with pytest.raises(MidtrainConfigError):
        check_linear_anneal_resume(cfg, 400_000_000_000)


class _Evil:
    def __reduce__(self):
        import os
        return (os.system, ("echo pwned > /dev/null",))


def test_untrusted_dcp_metadata_is_refused(tmp_path):
    d = tmp_path / "dcp"
    d.mkdir()
    (d / ".metadata").write_bytes(pickle.dumps(_Evil()))
    with pytest.raises(UntrustedCheckpointError):
        validate_dcp_metadata(d)
    (d / ".metadata").write_bytes(pickle.dumps({"x": eval}))
    with pytest.raises(UntrustedCheckpointError):
        validate_dcp_metadata(d)
    (d / ".metadata").write_bytes(b"not a pickle")
    with pytest.raises(UntrustedCheckpointError):
        validate_dcp_metadata(d)


def test_latest_ignores_incomplete_and_gc(tmp_path):
    ck = Checkpointer(tmp_path)
    for s in (1, 2, 3, 4, 5, 6):
        d = ck.step_dir(s)
        d.mkdir(parents=True)
        if s != 6:
            (d / "_COMPLETE").write_text("x")
    assert ck.latest() == ck.step_dir(5) and ck.complete_steps() == [1, 2, 3, 4, 5]
    ck.garbage_collect(keep_last=2, keep_every=0)
    assert ck.complete_steps() == [4, 5] and ck.step_dir(6).exists()


def test_stale_gradient_buffers_are_overwritten_not_accumulated_into(tmp_path):
    """``zero_grads`` writes nothing: the first micro-batch of a virtual rank stores its weight gradients and whatever
    no kernel wrote is zeroed afterwards; a second micro-batch accumulates. Poisoned buffers must not leak through."""
    import torch

    from helpers import tiny_cfg
    from open_transformers_b200.train.engine import TrainEngine

    cfg = tiny_cfg(str(tmp_path))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
    lab = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)

    def grads(poison: bool, micro_batches: int):
        eng = TrainEngine(cfg, "cpu")
        if poison:
            for buf in eng.grads:
                buf.fill_(123.0)
        eng.zero_grads()
        for _ in range(micro_batches):
            for v in range(len(eng.grads)):
                eng.forward_backward(v, ids, lab, micro_batches)
        out = [b.clone() for b in eng.grads]
        eng.close()
        return out

    clean1, dirty1 = grads(False, 1), grads(True, 1)
    assert all(torch.equal(a, b) for a, b in zip(clean1, dirty1))
    clean2, dirty2 = grads(False, 2), grads(True, 2)
    assert all(torch.equal(a, b) for a, b in zip(clean2, dirty2))
    # unseen vocabulary rows of the embedding table read zero, seen ones do not
    assert float(clean1[0].abs().sum()) > 0 and bool((clean1[0] == 0).any())


def test_grad_norm_log_folds_categories_and_blocks_from_per_tensor_norms(tmp_path):
    import json
    import math

    from helpers import tiny_cfg
    from open_transformers_b200.obs import grad_norm_log as GN
    from open_transformers_b200.train.loop import train

    names = ["embedding.tok_embeddings.weight", "blocks.0.attn.wq.weight", "blocks.0.attn.wq.weight_scale", "blocks.1.ffn.w_down.weight",
             "blocks.1.norm2.weight", "norm_out.weight", "embedding.output.weight"]
    assert [GN.category(n) for n in names] == ["embed", "attn", "lsq_scale", "ffn", "norm", "norm", "lm_head"]
    rec = GN.build_record(3, 99, names, [4.0, 9.0, 1.0, 16.0, 0.0, 1.0, 25.0], top_k=2)
    assert rec["global"] == round(math.sqrt(56.0), 6) and rec["by_layer"] == {"0": round(math.sqrt(10.0), 6), "1": 4.0}
    assert rec["by_category"]["norm"] == 1.0 and rec["top"] == [["embedding.output.weight", 5.0], ["blocks.1.ffn.w_down.weight", 4.0]]
    tmp = str(tmp_path)
    res = train(tiny_cfg(tmp, ["++train.grad_norm_log.every_n_steps=1", "++train.grad_norm_log.weight_stats_every_n_steps=2"]), device="cpu", data_root=tmp)
    rows = [json.loads(l) for l in open(res["run_dir"] + "/logs/grad_norms.jsonl")]
    assert [r["step"] for r in rows] == [1, 2, 3] and all(set(r) >= {"global", "by_category", "by_layer", "top"} for r in rows)
    metrics = [json.loads(l) for l in open(res["run_dir"] + "/logs/metrics.jsonl")]
    assert abs(rows[0]["global"] - metrics[0]["grad_norm_pre_clip"]) < 1e-4 * rows[0]["global"]
    assert "weight_norms" in rows[1] and "weight_norms" not in rows[0] and rows[1]["weight_norms"]["norm_out.weight"] > 0


def test_phase_timers_land_in_the_metrics_rows(tmp_path, monkeypatch):
    import json

    from helpers import tiny_cfg
    from open_transformers_b200.train.loop import train

    monkeypatch.setenv("PRETRAIN_CUDA_EVENT_TIMING", "1")
    tmp = str(tmp_path)
    res = train(tiny_cfg(tmp, []), device="cpu", data_root=tmp)
    rows = [json.loads(l) for l in open(res["run_dir"] + "/logs/metrics.jsonl")]
    for r in rows:
        assert all(r["phase_%s_ms" % k] > 0 for k in ("fwd", "bwd", "clip", "opt"))
        assert r["phase_fwd_ms"] + r["phase_bwd_ms"] + r["phase_clip_ms"] + r["phase_opt_ms"] <= r["step_wall_time_ms"]
    monkeypatch.delenv("PRETRAIN_CUDA_EVENT_TIMING")
    res2 = train(tiny_cfg(tmp + "/b", []), device="cpu", data_root=tmp + "/b")
    assert res2["hashes"] == res["hashes"]
    assert "phase_fwd_ms" not in json.loads(open(res2["run_dir"] + "/logs/metrics.jsonl").readline())


def test_parallel_dims_arithmetic():
    from open_transformers_b200.parallel import ParallelDims

    d = ParallelDims(1, 8, 2, 1, 8)                       # 8 virtual ranks (shard 8) on 2 processes
    assert (d.virtual_dp, d.dp_shard, d.dp_processes) == (8, 8, 2) and d.hosted_virtual_ranks(1) == [4, 5, 6, 7]
    d = ParallelDims(2, -1, 8, 2, 0)                      # 8 processes, tensor-parallel pairs: 4 data-parallel processes, 2 x 2
    assert (d.virtual_dp, d.dp_shard, d.dp_processes) == (4, 2, 4) and d.hosted_virtual_ranks(5) == [2] and d.tp_rank(5) == 1
    assert d.coords(3) == (1, 1)
    assert ParallelDims(2, -1, 1).virtual_dp == 2         # more replicas than processes: one process hosts both
    assert ParallelDims(1, -1, 1, 1, 6).dp_shard == 6
    for bad in ((1, 3, 2, 1, 4), (1, 4, 3, 1, 4), (1, 2, 3, 2, 0), (0, 1, 1)):
        with pytest.raises(ValueError):
            ParallelDims(*bad)


def test_metrics_logger_flushes_on_cadence_and_mirrors_to_the_tracker(tmp_path, monkeypatch):
    import json
    import sys
    import types

    from open_transformers_b200.obs.metrics import MetricsLogger, mfu, time_section, transformer_flops_per_token
    from open_transformers_b200.obs.wandb_run import WandBRun

    seen = []
    tracker = types.SimpleNamespace(log=lambda row, step=None: seen.append((step, row["loss"])))
    path = tmp_path / "logs" / "m.jsonl"
    lg = MetricsLogger(path, tracker, flush_every=3)
    for i in range(4):
        lg.log({"loss": float(i), "b": "x"}, step=i)
    assert len(path.read_text().splitlines()) == 3                 # flushed after the third row, the fourth still buffered
    lg.close()
    rows = [json.loads(l) for l in path.read_text().splitlines()]
    assert [r["loss"] for r in rows] == [0.0, 1.0, 2.0, 3.0] and seen == [(0, 0.0), (1, 1.0), (2, 2.0), (3, 3.0)]
    off = MetricsLogger(tmp_path / "no" / "m.jsonl", enabled=False)
    off.log({"loss": 1.0})
    off.close()
    assert not (tmp_path / "no").exists()
    sink = {}
    with time_section(sink, "a"):
        pass
    with time_section(sink, "a"):
        pass
    assert sink["a"] >= 0.0 and len(sink) == 1
    f = transformer_flops_per_token(24, 2048, 4096, 128256)
    assert f == 72 * 24 * 2048 ** 2 + 12 * 24 * 4096 * 2048 + 6 * 128256 * 2048 and abs(mfu(1e5, f, 2.25e15) - 1e5 * f / 2.25e15) < 1e-12
    # the tracker wrapper is a null object without credentials, with WANDB_MODE=disabled, and off rank 0
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    for kw, mode in (({}, ""), ({}, "disabled"), ({"enabled": False}, "offline")):
        monkeypatch.setenv("WANDB_MODE", mode)
        w = WandBRun("p", "r", **kw)
        w.log({"loss": 1.0}, step=1)
        w.finish()
        assert w._run is None
    # with a tracker module present and offline mode it initialises and forwards
    calls = []
    fake_run = types.SimpleNamespace(log=lambda row, step=None: calls.append(("log", step)), finish=lambda: calls.append(("finish", None)))
    monkeypatch.setitem(sys.modules, "wandb", types.SimpleNamespace(init=lambda **kw: (calls.append(("init", kw["project"])), fake_run)[1]))
    monkeypatch.setenv("WANDB_MODE", "offline")
    w = WandBRun("proj", "run1")
    w.log({"loss": 2.0}, step=5)
    w.finish()
    assert calls == [("init", "proj"), ("log", 5), ("finish", None)]


@pytest.mark.parametrize("bf16", [False, True])
def test_activation_checkpointing_changes_no_bit(bf16, monkeypatch):
    """recompute runs the same deterministic kernels: every block, every other block and no checkpointing give one hash;
    and it really recomputes (the block forward runs again during the backward pass)"""
    from open_transformers_b200.config import load_config
    from open_transformers_b200.ops import functional as K
    from open_transformers_b200.train.engine import TrainEngine

    def run(extra):
        cfg = load_config("tiny_cpu", ["model.n_layers=3", "run.mixed_precision=%s" % ("true" if bf16 else "false"), *extra])
        eng = TrainEngine(cfg, "cpu")
        g = torch.Generator().manual_seed(0)
        calls = {"n": 0}
        orig = K.rmsnorm_fwd

        def counted(*a, **k):
            calls["n"] += 1
            return orig(*a, **k)

        monkeypatch.setattr(K, "rmsnorm_fwd", counted)      # two norms per block and the final one, per forward pass
        eng.zero_grads()
        for v in range(eng.V):
            ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
            eng.forward_backward(v, ids, torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), 1)
        norm = eng.reduce_gradients()
        eng.optimizer_step(1e-3, 1.0)
        h = eng.sharded_state_hash(None, None)
        monkeypatch.setattr(K, "rmsnorm_fwd", orig)
        eng.close()
        return h, norm, calls["n"]

    plain = run(["run.activation_checkpoint=false"])
    every = run(["run.activation_checkpoint=true"])
    other = run(["run.activation_checkpoint=true", "run.ac_every_other_block=true"])
    assert plain[:2] == every[:2] == other[:2]
    per_pass = 2 * 3 + 1
    assert plain[2] == 2 * per_pass and every[2] == 2 * (per_pass + 6) and other[2] == 2 * (per_pass + 4)   # blocks 0 and 2 of 3 recomputed


def test_cpu_attention_results_survive_the_recomputation_when_asked(monkeypatch):
    """PRETRAIN_CPU_ATTENTION_CHECKPOINT_CACHE=1: under activation checkpointing on a CPU the recomputed block forward takes
    each attention result from the original forward pass instead of running the kernel again; same hash, fewer calls."""
    from open_transformers_b200.config import load_config
    from open_transformers_b200.ops import autograd as A
    from open_transformers_b200.ops import functional as K
    from open_transformers_b200.train.engine import TrainEngine

    def run(cache):
        if cache:
            monkeypatch.setenv("PRETRAIN_CPU_ATTENTION_CHECKPOINT_CACHE", "1")
        else:
            monkeypatch.delenv("PRETRAIN_CPU_ATTENTION_CHECKPOINT_CACHE", raising=False)
        cfg = load_config("tiny_cpu", ["model.n_layers=3", "run.activation_checkpoint=true"])
        eng = TrainEngine(cfg, "cpu")
        g = torch.Generator().manual_seed(0)
        calls = {"n": 0}
        orig = K.attn_fwd

        def counted(*a, **k):
            calls["n"] += 1
            return orig(*a, **k)

        monkeypatch.setattr(K, "attn_fwd", counted)
        hits0 = A._attn_cache["hits"]
        eng.zero_grads()
        for v in range(eng.V):
            ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
            eng.forward_backward(v, ids, torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), 1)
        norm = eng.reduce_gradients()
        eng.optimizer_step(1e-3, 1.0)
        h = eng.sharded_state_hash(None, None)
        monkeypatch.setattr(K, "attn_fwd", orig)
        eng.close()
        return h, norm, calls["n"], A._attn_cache["hits"] - hits0

    plain, cached = run(False), run(True)
    assert plain[:2] == cached[:2]
    assert plain[2] == 2 * 2 * 3 and plain[3] == 0            # two virtual ranks x (forward + recomputation) x three blocks
    assert cached[2] == 2 * 3 and cached[3] == 2 * 3          # the recomputation took all six results from the first pass
    assert A._attn_cache["mode"] is None


@pytest.mark.parametrize("bf16", [False, True])
def test_training_step_hash_is_the_same_on_the_plain_and_the_lane_parallel_gemm_twins(bf16):
    from open_transformers_b200.config import load_config
    from open_transformers_b200.ops.native import cpu_lib
    from open_transformers_b200.train.engine import TrainEngine

    def run():
        cfg = load_config("tiny_cpu", ["run.mixed_precision=%s" % ("true" if bf16 else "false")])
        eng = TrainEngine(cfg, "cpu")
        g = torch.Generator().manual_seed(0)
        prev = None
        for _ in range(2):
            eng.zero_grads()
            for v in range(eng.V):
                ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
                eng.forward_backward(v, ids, torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), 1)
            norm = eng.reduce_gradients()
            eng.optimizer_step(1e-3, eng.clip_coefficient(norm, 1.0))
            prev = eng.sharded_state_hash(prev, None)
        eng.close()
        return prev

    lib = cpu_lib()
    lib.otb_cpu_gemm_set_plain(1)
    try:
        plain = run()
    finally:
        lib.otb_cpu_gemm_set_plain(0)
    assert run() == plain
