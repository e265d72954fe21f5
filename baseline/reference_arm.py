"""Reference arm of `bench.py`: the unmodified reference harness, timed on the same box and config.

What runs is the reference's own `pretrain.train.loop.train(cfg)` from `baseline/_ref` (a plain copy of the
reference's `src/pretrain` and `configs`): its model, FSDP2 wrap, deterministic reduce-scatter, global-norm
clip, per-parameter AdamW loop, canonical data stream, per-step state hash and metrics. The only things that
are not the reference's are the libraries underneath it, which do not exist on this image:

* `repop` (closed source) -> `baseline/shims/repop`, every entry point on the fastest stock path of the box
  (cuBLAS, FlashAttention-2, `F.rms_norm`, `F.silu`, `nn.Embedding`, PyTorch's fused AdamW kernel);
* `hydra-core` / `omegaconf` -> `baseline/shims/hydra`, `baseline/shims/omegaconf` (YAML composition only).

Nothing of `open_transformers_b200` is imported and none of its native libraries is loaded.

Timing. `train()` offers no "run K steps and tell me how long" call, so the harness wraps the one function the
loop calls at the top of every optimizer step on every rank (`schedule_lr`). At the start of step W it runs a
barrier and a device synchronise and records a CUDA event; at the start of step W+K it records the second
event, synchronises, takes the maximum over ranks and stops the run by raising through `train()`'s own
`finally` (which closes the logs and the process group). The K timed steps therefore contain everything the
reference does per step: host-to-device copies of every micro-batch from pinned memory, the loss read-back per
micro-batch, the gradient reduction, clip, optimizer, the state hash (device-to-host copy of the local state +
blake2b on the host) and the metrics line. There is no second, device-resident-input mode in the reference's
loop, so `value` and `e2e.value` are the same measurement.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = Path(os.environ.get("OTB_REFERENCE_DIR", str(HERE / "_ref")))
SHIMS = HERE / "shims"
METRIC = "OPEN-1B training tokens/s (bit-identical step hash across GPU counts)"


class _BenchDone(BaseException):
    """Raised at the top of step W+K to leave `train()` through its own cleanup."""


class _Clocks:
    """nvidia-smi SM clock and throttle-reason samples of one GPU while the steps are timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.5)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def install_hint() -> str | None:
    """None when the reference copy and the stand-ins are in place, else the reason they are not."""
    if not (REF / "pretrain" / "train" / "loop.py").is_file() or not (REF / "configs" / "train").is_dir():
        return "baseline/_ref holds no copy of the reference (run `python baseline/install_reference.py <reference checkout>`)"
    if not (SHIMS / "repop" / "__init__.py").is_file():
        return "baseline/shims/repop is missing"
    return None


def _print_unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def run(gpus: int, steps: int, warmup: int, overrides: list[str] | None = None, tiny: bool = False) -> int:
    """Time K steps of the reference's `train()`; rank 0 prints the bench line. `tiny` (tests only) swaps the
    OPEN-1B model for a two-layer one so the whole path can run on CPU ranks."""
    why = install_hint()
    if why:
        return _print_unavailable(why)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ and not tiny:
        # the reference is always started by torchrun (scripts/launch_single_node.sh), also on one GPU: its device mesh
        # needs a process group. A bare `python bench.py --impl reference` gets the environment of a one-rank launch.
        os.environ.update({"RANK": "0", "WORLD_SIZE": "1", "LOCAL_RANK": "0"})
        os.environ.setdefault("MASTER_PORT", str(29600 + os.getpid() % 2000))
    for p in (str(SHIMS), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    for name in list(sys.modules):
        if name == "open_transformers_b200" or name.startswith("open_transformers_b200."):
            return _print_unavailable("open_transformers_b200 was imported before the reference arm started")

    import logging

    import torch

    logging.basicConfig(level=logging.WARNING)
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not use_cuda and not tiny:
        return _print_unavailable("no CUDA device is visible: the OPEN-1B-sized reference step is only timed on a GPU")
    if world != gpus and not tiny:
        return _print_unavailable("--gpus %d needs a torch.distributed.run launch with %d ranks (got WORLD_SIZE=%d)" % (gpus, gpus, world))

    V, mb, T = 8, 4, 4096                      # 8 micro-batches of 4 x 4096 tokens per optimizer step, whatever N is
    vocab = 128256
    if tiny:
        V, mb, T, vocab = max(2, world), 2, 128, 1024
    tokens_per_step = V * mb * T
    if V % world:
        return _print_unavailable("the step's %d micro-batches do not divide over %d ranks" % (V, world))
    n_steps = warmup + steps

    # synthetic uniform-random token shards, written by the reference's own `prepare-data synthetic` tool
    work = Path(tempfile.mkdtemp(prefix="ref_arm_r%d_" % rank))
    data_dir = work / "shards"
    need = (n_steps + 2) * tokens_per_step * 2
    max_len = 8192 if not tiny else 512
    docs_a = max(64, need // (max_len // 2))
    from pretrain.cli import prepare_data as _prep

    argv, sys.argv = sys.argv, ["prepare_data", "synthetic", "--output-dir", str(data_dir), "--docs-a", str(docs_a), "--docs-b", "64",
                                "--min-doc-len", str(max_len // 4), "--max-doc-len", str(max_len), "--vocab-size", str(vocab), "--seed", "0"]
    try:
        _prep.main()
    finally:
        sys.argv = argv

    from pretrain.config import load_config

    ov = [
        "model.qat.enabled=false", "model.attn_int8_pv=false", "model.emb_norm=false", "model.qk_norm_gain=false",
        "model.z_loss.coeff=1.0e-4",
        "run.dp_shard_size=-1", "run.dp_replicate_size=1", "run.seed=0", "run.output_dir=%s" % (work / "runs"), "run.run_id=bench",
        "run.mixed_precision=true", "run.reduction_mode=deterministic_allgather",
        # 180 GB parts hold every activation of a 16 384-token micro-batch: recompute off is the faster stock setting
        "run.activation_checkpoint=%s" % os.environ.get("REF_ARM_ACTIVATION_CHECKPOINT", "false"),
        "data.sources=[{name: synth_a, path: %s, weight: 0.7}, {name: synth_b, path: %s, weight: 0.3}]" % (data_dir / "synth_a", data_dir / "synth_b"),
        "data.seq_len=%d" % T, "+data.weights_are_token_shares=false",
        "train.seq_len=%d" % T, "train.micro_batch_size=%d" % mb,
        "train.total_tokens=%d" % ((n_steps + 1) * tokens_per_step),
        "train.global_batch_tokens.warmup=%d" % tokens_per_step, "train.global_batch_tokens.main=%d" % tokens_per_step,
        "train.global_batch_tokens.late=%d" % tokens_per_step,
        "train.warmup_to_main_at_tokens=0", "train.main_to_late_at_tokens=0",
        "train.ckpt_every_steps=1000000", "train.state_hash.every_n_steps=1",
    ]
    if tiny:
        ov += ["model.n_layers=2", "model.d_model=128", "model.n_heads=4", "model.n_kv_heads=2", "model.head_dim=32",
               "model.ffn_intermediate=256", "model.vocab_size=%d" % vocab, "model.max_seq_len_pretrain=%d" % T, "model.swa_window=64",
               "model.swa_full_every=2"]
    cfg = load_config("1b_repop_v2", ov + list(overrides or []))

    import pretrain.train.loop as loop_mod

    state = {"i": 0, "e0": None, "ms": None, "clocks": None, "sampler": None, "n_params": 0}
    inner = loop_mod.schedule_lr
    inner_build_optimizer = loop_mod.build_optimizer

    def counting_build_optimizer(model, optim_cfg):
        state["n_params"] = sum(int(p.numel()) for p in model.parameters())
        return inner_build_optimizer(model, optim_cfg)

    def _sync():
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    def hooked_schedule_lr(optimizer, lr):
        i = state["i"]
        if i == warmup:
            _sync()
            if use_cuda:
                state["e0"] = torch.cuda.Event(enable_timing=True)
                state["e0"].record()
            import time

            state["t0"] = time.perf_counter()
            if use_cuda:
                state["sampler"] = _Clocks(local_rank)
                state["sampler"].start()
        elif i == warmup + steps:
            import time

            if use_cuda:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                torch.cuda.synchronize()
                ms = state["e0"].elapsed_time(e1)
            else:
                ms = (time.perf_counter() - state["t0"]) * 1e3
            state["wall_ms"] = (time.perf_counter() - state["t0"]) * 1e3
            if state["sampler"] is not None:
                state["clocks"] = state["sampler"].stop()
            if torch.distributed.is_available() and torch.distributed.is_initialized():
                t = torch.tensor([ms], dtype=torch.float64, device="cuda" if use_cuda else "cpu")
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
                ms = float(t.item())
            state["ms"] = ms
            raise _BenchDone()
        state["i"] = i + 1
        return inner(optimizer, lr)

    loop_mod.schedule_lr = hooked_schedule_lr
    loop_mod.build_optimizer = counting_build_optimizer
    try:
        try:
            loop_mod.train(cfg)
        except _BenchDone:
            pass
    except torch.OutOfMemoryError as e:  # pragma: no cover - needs a GPU
        return _print_unavailable("the reference loop ran out of device memory: %s" % str(e).splitlines()[0])
    finally:
        loop_mod.schedule_lr = inner
        loop_mod.build_optimizer = inner_build_optimizer
    if state["ms"] is None:
        return _print_unavailable("the reference loop ended before step %d" % (warmup + steps))

    if rank == 0:
        ms = state["ms"]
        tps = tokens_per_step * steps / (ms / 1e3)
        # the reference's own per-step records of the timed steps (rank 0's metrics.jsonl)
        rows = []
        mpath = work / "runs" / "bench" / cfg.logging.metrics_jsonl_path
        if mpath.is_file():
            for ln in mpath.read_text().splitlines():
                try:
                    r = json.loads(ln)
                except Exception:
                    continue
                if warmup < r.get("step", 0) <= warmup + steps:
                    rows.append(r)
        hashes = []
        hpath = work / "runs" / "bench" / "logs" / "state_hashes.jsonl"
        if hpath.is_file():
            hashes = [json.loads(ln) for ln in hpath.read_text().splitlines() if ln.strip()]
        compute_ms = statistics.mean(r["step_compute_time_ms"] for r in rows) if rows else None
        hash_ms = statistics.mean(r["hash_time_ms"] for r in rows) if rows else None
        accum = V // world
        line = {
            "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"model": cfg.model.name, "params": state["n_params"], "global_batch": V * mb, "seq_len": T, "global_batch_tokens": tokens_per_step,
                       "parallelism": "reference FSDP2 shard group of %d (no wrap at 1 rank), gradient accumulation %d, deterministic_allgather reduce-scatter" % (world, accum),
                       "l2": "inputs larger than L2 (fp32 / bf16 weights of 1.6 B parameters per micro-batch)",
                       "state_hash": "every step: reference's host blake2b over the local state",
                       "activation_checkpoint": cfg.run.activation_checkpoint,
                       "harness": "unmodified reference train() from baseline/_ref over the stock-torch repop stand-in"},
            "clocks": state["clocks"],
            "e2e": {"value": tps, "unit": "tokens/s", "ms_per_step": ms / steps,
                    "h2d_bytes_per_step": V * mb * T * 8 * 2, "d2h_bytes_per_step": 8 * V + 16 * state["n_params"],
                    "note": "the reference loop has one mode: pinned-host batches copied in and losses read back every micro-batch; "
                            "its state hash copies the whole training state (fp32 weights, two moments, gradients: 16 bytes per parameter over all ranks) to the host every step"},
            "gpu_launches": 0,
            "reference_step_records": {"n": len(rows), "mean_step_compute_time_ms": compute_ms, "mean_hash_time_ms": hash_ms,
                                       "tokens_per_s_without_hash_and_logging": (tokens_per_step / (compute_ms / 1e3)) if compute_ms else None},
            "final_loss": rows[-1]["loss_ce"] if rows else None,
            "final_hash": hashes[-1]["state_hash"] if hashes else None,
            "wall_ms_per_step": state.get("wall_ms", 0.0) / steps,
        }
        print(json.dumps(line), flush=True)
    import shutil

    shutil.rmtree(work, ignore_errors=True)
    return 0
