"""Headline benchmark: OPEN-1B-shaped pretraining step throughput (tokens/s) on N B200 GPUs of one node.

  python bench.py --gpus 1 --steps 3 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
         bench.py --gpus N --steps K --warmup W

One step = the full optimizer step of the `open1b_b200` recipe: 8 virtual ranks x 4 sequences x
4096 tokens (131 072 tokens, fixed whatever N is: strong scaling), forward + backward through the
native sm_100a kernels, deterministic gradient reduction, global-norm clip, AdamW, weight
redistribution and the chained state hash (tree digests on the device). Random-init weights
(Philox, seed 0), synthetic uniform-random tokens (seed 0).

Two timed regions of K steps each, both on the device with CUDA events, max over ranks:
  * `value`: inputs already resident on the device;
  * `e2e`:   the calls `train()` makes: micro-batches come from the canonical data stream over synthetic shards
             (`build_global_loader`), are collated into pinned host memory, chained into the per-virtual-rank batch
             digests and copied to the device inside the timed region; the step's loss is read back to the host and
             the batch digest goes into the state hash every step.
`--impl reference` times the unmodified reference training loop (`baseline/_ref`) over a stock-torch stand-in of
its closed kernel library, same config, steps and warm-up (`baseline/reference_arm.py`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput figure


class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, sampled every 200 ms while a region is timed. Reads NVML in this
    process (the library behind nvidia-smi; a read costs microseconds and starts no process next to the timed kernels);
    without the Python binding it falls back to ONE long-running ``nvidia-smi -lms 200`` for the region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int, uuid: str | None = None):
        self.index, self.uuid, self.rows, self._stop, self._t, self._proc = index, uuid, [], threading.Event(), None, None
        self._nvml = self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid) if uuid else pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n, h = self._nvml, self._handle
        bits = n.nvmlDeviceGetCurrentClocksEventReasons(h)
        masks = (n.nvmlClocksEventReasonHwSlowdown, n.nvmlClocksEventReasonHwThermalSlowdown, n.nvmlClocksEventReasonSwThermalSlowdown,
                 n.nvmlClocksEventReasonSwPowerCap)
        return [str(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)), str(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)),
                "%.1f" % (n.nvmlDeviceGetPowerUsage(h) / 1e3)] + ["Active" if bits & m else "Not Active" for m in masks]

    def _run(self):
        while not self._stop.is_set():
            try:
                self.rows.append(self._sample_nvml())
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        if self._nvml is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
            return
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid or str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                           "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None

    def stop(self) -> dict:
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        if self._proc is not None:
            self._proc.terminate()  # the one process this sampler started
            try:
                out, _ = self._proc.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
                out, _ = self._proc.communicate()
            self.rows += [[c.strip() for c in line.split(",")] for line in out.splitlines() if line.strip()]
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        watts = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, val in zip(self.REASONS, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": statistics.median(watts) if watts else None, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvml" if self._nvml is not None else "nvidia-smi"}


def reference_arm(args) -> int:
    """The unmodified reference training loop over a stock-torch stand-in of its closed kernel library
    (`baseline/reference_arm.py`); imports nothing of this package."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("reference_arm", os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "reference_arm.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.run(args.gpus, args.steps, args.warmup, tiny=os.environ.get("OTB_REFERENCE_ARM_TINY") == "1")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="open1b_b200")
    ap.add_argument("--override", action="extend", nargs="+", default=[], help="config override (debugging; makes the number invalid)")
    ap.add_argument("--no-hash", action="store_true", help="debugging: skip the per-step state hash (makes the number invalid)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel group size (run.tp_size); the GPUs form one group")
    ap.add_argument("--tp-fused", action="store_true", help="with --tp: peer-memory all-gather->GEMM / chained GEMM kernels (run.tp_fused)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from open_transformers_b200.config import load_config
    from open_transformers_b200.ops import native
    from open_transformers_b200.ops.functional import kernel_status
    from open_transformers_b200.optim.schedules import build_schedule
    from open_transformers_b200.train.engine import TrainEngine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs a torch.distributed.run launch with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    native.cuda_lib()

    cfg = load_config(args.config, args.override + (["run.tp_size=%d" % args.tp] if args.tp > 1 else [])
                      + (["run.tp_fused=true"] if args.tp_fused else []))
    V = cfg.run.virtual_dp_size
    eng = TrainEngine(cfg, device, rank, world, None)
    mb, T = cfg.train.micro_batch_size, cfg.train.seq_len
    accum = max(1, cfg.train.global_batch_tokens.main // (mb * T * V))
    tokens_per_step = V * accum * mb * T
    sched = build_schedule(cfg.schedule, cfg.train, cfg.optim)
    vocab = cfg.model.vocab_size
    hosted = eng.hosted
    total_steps = 2 * (args.steps + args.warmup)

    # synthetic uniform-random tokens from seed 0: stream position = (step, virtual rank, micro-batch)
    def host_batch(step: int, v: int, k: int):
        g = torch.Generator().manual_seed((step * V + v) * accum + k)
        seq = torch.randint(0, vocab, (mb, T + 1), generator=g, dtype=torch.int64)
        return seq[:, :-1].contiguous().pin_memory(), seq[:, 1:].contiguous().pin_memory()

    host = {(s, v, k): host_batch(s, v, k) for s in range(args.steps + args.warmup) for v in hosted for k in range(accum)}
    h2d_bytes = sum(a.numel() * 8 + b.numel() * 8 for (s, v, k), (a, b) in host.items() if s == 0)
    state = {"prev": None, "consumed": 0, "step": 0, "loss": None, "pending": None, "pending_bd": None}

    # the end-to-end region reads the canonical stream: seed-generated shards, written once by rank 0
    import tempfile

    from open_transformers_b200.data.loader import build_global_loader, collate
    from open_transformers_b200.data.synthetic import ensure_synthetic_sources
    from open_transformers_b200.train import state_hash as SH

    data_root = os.path.join(tempfile.gettempdir(), "otb_bench_data_%s_%d" % (os.environ.get("MASTER_PORT", "single"), os.getppid() if world > 1 else os.getpid()))
    if rank == 0:
        ensure_synthetic_sources(cfg, data_root, (args.steps + args.warmup + 2) * tokens_per_step)
    if world > 1:
        dist.barrier()
    stream = iter(build_global_loader(cfg, hosted, V, data_root=data_root))
    hashers = {v: SH.RunningBatchHasher() for v in hosted}

    def batch_digest():
        chains = {v: h.local_digest() for v, h in hashers.items()}
        if world > 1:
            objs = [None] * world
            dist.all_gather_object(objs, chains, group=eng.host_group)  # host bytes over gloo: no wait on the device's queue
            chains = {k: d for part in objs for k, d in part.items()}
        return SH.combine_batch_digests([chains[v] for v in range(V)])

    def one_step(step: int, resident):
        eng.zero_grads()
        last_ce = None
        bd = None
        if resident is not None:
            for vi, v in enumerate(hosted):
                for k in range(accum):
                    ids, labels = resident[(step, v, k)]
                    ce, z = eng.forward_backward(vi, ids, labels, accum, last=(vi == len(hosted) - 1 and k == accum - 1))
                    last_ce = ce
        else:
            plan, batches = next(stream)
            batches = list(batches)
            for j, (v, k, windows) in enumerate(batches):
                batch = collate(windows, pin=True)
                hashers[v].update(batch)
                ids, labels = batch["input_ids"].to(device, non_blocking=True), batch["labels"].to(device, non_blocking=True)
                ce, z = eng.forward_backward(hosted.index(v), ids, labels, accum, last=j == len(batches) - 1)
                last_ce = ce
            bd = batch_digest()
        if not args.no_hash:
            flush_hash()  # the previous step's digests ran under this step's forward/backward; fold them in while it drains
        norm = eng.reduce_gradients()
        lr = sched(state["consumed"], cfg.train.total_tokens)
        eng.optimizer_step(lr, eng.clip_coefficient(norm, cfg.train.grad_clip))
        state["consumed"] += tokens_per_step
        if not args.no_hash:
            # the digests of this step's state run on a side stream under the next step's forward/backward
            state["pending"] = eng.begin_state_hash(include_grads=cfg.train.state_hash.include_grads)
            state["pending_bd"] = bd
        return last_ce, norm

    def flush_hash():
        if state.get("pending") is not None:
            state["prev"] = eng.finish_state_hash(state["pending"], state["prev"], state["pending_bd"])
            state["pending"] = None

    def timed(first_step: int, n: int, resident_mode: bool):
        resident = None
        if resident_mode:
            resident = {(s, v, k): (host[(s, v, k)][0].to(device), host[(s, v, k)][1].to(device))
                        for s in range(first_step, first_step + n) for v in hosted for k in range(accum)}
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = None
        for s in range(first_step, first_step + n):
            ce, norm = one_step(s, resident)
            if not resident_mode:
                loss = float(ce.detach().to("cpu"))  # the step's result is read on the host every step
        flush_hash()  # every hash of the timed steps completes inside the timed region
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, loss

    W, Kst = args.warmup, args.steps
    timed(0, W, True)                       # warm-up (untimed)
    sampler = ClockSampler(local_rank, "GPU-%s" % torch.cuda.get_device_properties(device).uuid)
    launches0 = native.launch_count
    sampler.start()
    eng.phase_report()                      # (phase timers, when PRETRAIN_CUDA_EVENT_TIMING=1: start from zero)
    ms_dev, _ = timed(W, Kst, True)
    phases = {k: v / Kst for k, v in eng.phase_report().items()}
    launches = native.launch_count - launches0
    clocks = sampler.stop()
    timed(0, W, False)                      # warm-up of the end-to-end path (the stream supplies its own batches)
    ms_e2e, loss = timed(0, Kst, False)
    status = kernel_status(device)
    if world > 1:
        dist.barrier()
    if rank == 0:
        import shutil

        shutil.rmtree(data_root, ignore_errors=True)
        tps = tokens_per_step * Kst / (ms_dev / 1e3)
        tps_e2e = tokens_per_step * Kst / (ms_e2e / 1e3)
        from open_transformers_b200.obs.metrics import hardware_flops_per_token

        hw_flops = hardware_flops_per_token(cfg.model, T)
        flops_per_token = 72 * cfg.model.n_layers * cfg.model.d_model ** 2 + 12 * cfg.model.n_layers * T * cfg.model.d_model + 6 * vocab * cfg.model.d_model
        line = {
            "metric": "OPEN-1B training tokens/s (bit-identical step hash across GPU counts)", "value": tps, "unit": "tokens/s",
            "n_gpus": world, "steps": Kst, "warmup": W, "ms_per_step": ms_dev / Kst, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (tps / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": cfg.model.name, "params": eng.layout.total, "global_batch": V * accum * mb, "seq_len": T,
                       "global_batch_tokens": tokens_per_step, "parallelism": "virtual dp8 (shard 8) on %d GPU(s)%s" % (world, ", tensor-parallel groups of %d" % args.tp if args.tp > 1 else ""),
                       "l2": "inputs larger than L2 (3.2 GB of bf16 weights + 6.4 GB fp32 gradients per micro-batch)",
                       "state_hash": "none" if args.no_hash else "every step, tree digests on device",
                       "e2e_path": "GlobalStream loader over synthetic shards -> pinned collate -> batch digests -> H2D, loss D2H per step",
                       "overrides": args.override},
            "clocks": clocks,
            "e2e": {"value": tps_e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / Kst,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4 + 4 * eng.n_segs},
            "gpu_launches": launches,
            # the reference's formula (every layer as dense T x T attention) and what the kernels execute (causal, 512-key windows)
            "model_tflops_per_gpu": flops_per_token * tps / world / 1e12,
            "hardware_flops_per_token": hw_flops, "hardware_tflops_per_gpu": hw_flops * tps / world / 1e12,
            "final_loss": loss, "final_hash": state["prev"], "kernel_status": status,
            "native_libs": native.loaded_libraries(),
        }
        if phases:  # diagnostic run with phase timers: device time per step inside forward / backward / reduction+norm / update
            line["phases_ms_per_step"] = phases
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
