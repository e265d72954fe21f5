"""``train(cfg, resume_from)``: the pre-training driver.

Per optimizer step (cf. reference src/pretrain/train/loop.py:789-1242): take the step's plan from the canonical
stream; every process runs the micro-batches of the virtual ranks it hosts (batch hashed on the CPU, copied
to the device, forward + backward); deterministic gradient reduction + global norm; spike decision on the
globally folded loss and the pre-clip norm; clip + AdamW (or skip); token / step counters; SIGTERM poll; state
hash when due (cadence, checkpoint, exit or final step - only cadence hashes advance the chain); checkpoint
when due; metrics. Gradients are zeroed only at the start of the next step, so the hash sees the post-clip
gradients of the step it describes.

Run directory ``<output_dir>/<run_id>/``: ``checkpoints/``, ``checkpoints/state_hash_init.txt``,
``logs/metrics.jsonl``, ``logs/state_hashes.jsonl``, ``logs/grad_norms.jsonl``.
"""
from __future__ import annotations

import json
import math
import logging
import os
import signal
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ..config.schema import RootConfig
from ..data.global_stream import GlobalStreamState
from ..data.loader import build_global_loader, collate
from ..obs.metrics import MetricsLogger, mfu, transformer_flops_per_token
from ..obs.wandb_run import WandBRun
from ..optim.schedules import build_schedule, rewarm_factor
from ..parallel.env import init_distributed, set_seed
from ..utils.git import git_sha, native_source_digests
from . import state_hash as SH
from .checkpoint import CheckpointMeta, Checkpointer, resolved_config_json
from .engine import TrainEngine
from .midtrain import check_linear_anneal_resume
from .qk_gain_control import clamp_qk_gains
from .spike_protocol import Halt, SpikeProtocol

log = logging.getLogger("pretrain.train")
_sigterm = {"flag": False}


def _on_sigterm(signum, frame):
    _sigterm["flag"] = True


def _emergency_exit_requested(world: int, device: torch.device, group=None) -> bool:
    """Every rank learns whether ANY rank received SIGTERM, so that all of them checkpoint at the same step. ``group``: a
    host-side (gloo) group, where there is one, so that the question does not wait for the device's queue."""
    if world == 1:
        return _sigterm["flag"]
    host = group is not None and dist.get_backend(group) == "gloo"
    t = torch.tensor([1 if _sigterm["flag"] else 0], dtype=torch.int32, device="cpu" if host else device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group if host else None)
    return bool(t.item())


def deterministic_scalar_sums(lists: dict[str, list[float]], world: int, group=None) -> dict[str, tuple[float, int]]:
    """Per key: sum and count of the python floats contributed by all ranks, folded in fp64 in rank order (telemetry and
    spike input). One exchange for all keys."""
    parts = [{k: [float(x) for x in v] for k, v in lists.items()}]
    if world > 1:
        parts = [None] * world
        dist.all_gather_object(parts, {k: [float(x) for x in v] for k, v in lists.items()}, group=group)
    out = {}
    for key in lists:
        total, n = 0.0, 0
        for part in parts:
            for v in part[key]:
                total += float(v)
                n += 1
        out[key] = (total, n)
    return out


def deterministic_scalar_sum(values: list[float], world: int, group=None) -> tuple[float, int]:
    """Sum of python floats contributed by all ranks, folded in fp64 in rank order."""
    return deterministic_scalar_sums({"x": values}, world, group)["x"]


def _assert_same_on_all_ranks(payload: str, what: str, world: int) -> None:
    if world == 1:
        return
    objs: list = [None] * world
    dist.all_gather_object(objs, payload)
    if len(set(objs)) != 1:
        raise RuntimeError("%s differs between ranks: %s" % (what, sorted(set(objs))))


def cross_entropy_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of full-vocabulary logits in the canonical summation order (no z-loss, no gradient side effects).
    The step itself uses the fused CE + z-loss; this is the plain form. (reference src/pretrain/train/loop.py:155-169)"""
    from ..models.fused_loss import cross_entropy

    return cross_entropy(logits, labels)


def _append_jsonl(path: Path, row: dict) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "a", encoding="utf-8") as f:
        f.write(json.dumps(row, sort_keys=True) + "\n")


def train(cfg: RootConfig, resume_from: str | None = None, *, device: str | None = None, data_root: str | None = None,
          max_steps: int | None = None) -> dict:
    rank, world, dev = init_distributed(device)
    signal.signal(signal.SIGTERM, _on_sigterm)
    _sigterm["flag"] = False
    set_seed(cfg.run.seed, rank)
    run_id = cfg.run.run_id or os.environ.get("RUN_ID", "run")
    _assert_same_on_all_ranks(run_id, "run_id", world)
    run_dir = Path(cfg.run.output_dir) / run_id
    ckpt = Checkpointer(run_dir, rank, world)
    if resume_from is None and ckpt.complete_steps():
        raise RuntimeError("%s already holds checkpoints; pass --resume-from or choose a new run_id (cold-start overwrite guard)" % run_dir)

    engine = TrainEngine(cfg, dev, rank, world)
    if cfg.train.ckpt_every_steps > 0 or cfg.train.ckpt_every_tokens > 0:
        ckpt.prepare(engine)  # page-lock the staging buffers before the first step, not inside the first checkpoint
    V, hosted = engine.V, engine.hosted
    if rank == 0:
        rb = engine.resident_bytes()
        log.info("training state per process: %.2f GiB (%s); %d virtual ranks hosted; gradient transport %s", rb["total"] / 2 ** 30,
                 ", ".join("%s %.2f" % (k, v / 2 ** 30) for k, v in rb.items() if k != "total" and v), len(hosted), engine.transport)
    train_cfg = cfg.train
    sched = build_schedule(cfg.schedule, train_cfg, cfg.optim)
    spike = SpikeProtocol.from_config(train_cfg.spike)
    hashers = {v: SH.RunningBatchHasher() for v in hosted}
    consumed, step, chained, restart_count, rewarm_anchor = 0, 0, None, 0, None
    stream_state = None

    if resume_from is not None:
        meta0 = Checkpointer.read_meta(resume_from)
        check_linear_anneal_resume(cfg, meta0.consumed_tokens)
        if (meta0.dp_world_size, meta0.dp_shard, meta0.dp_replicate) != (V, engine.dp_shard, engine.dp_replicate):
            raise RuntimeError("checkpoint was written for virtual topology %s, this run uses %s (a different topology starts a new segment)"
                               % ((meta0.dp_world_size, meta0.dp_shard, meta0.dp_replicate), (V, engine.dp_shard, engine.dp_replicate)))
        side = ckpt.load(resume_from, engine, load_optimizer=not train_cfg.resume_reset_optimizer)
        consumed, step, chained = meta0.consumed_tokens, meta0.step, meta0.chained_hash
        restart_count = meta0.restart_count + 1
        stream_state = GlobalStreamState.from_json(side["global_stream"]) if side["global_stream"] else None
        spike.load_state_dict(side["spike_protocol"])
        hashers = {v: SH.RunningBatchHasher(side["batch_chains"][v]) for v in hosted}
        # LR re-warm anchor (reference src/pretrain/train/loop.py:565-586): a resume that resets the optimizer ramps from the
        # resume point; a moments-kept resume with rewarm_on_resume continues a recorded ramp, or starts one here; else none
        if train_cfg.resume_reset_optimizer:
            rewarm_anchor = consumed
        elif cfg.schedule.rewarm_on_resume and cfg.schedule.rewarm_tokens > 0:
            prev = meta0.rewarm_anchor_tokens
            rewarm_anchor = prev if (prev is not None and prev >= 0) else consumed
        else:
            rewarm_anchor = None
    else:
        check_linear_anneal_resume(cfg, None)

    loader = build_global_loader(cfg, hosted, V, state=stream_state, consumed_tokens=consumed, start_step=step, data_root=data_root)
    metrics = MetricsLogger(run_dir / cfg.logging.metrics_jsonl_path, WandBRun(cfg.logging.wandb_project, run_id, enabled=rank == 0),
                            enabled=rank == 0)
    hash_log = run_dir / "logs" / "state_hashes.jsonl"
    gn_log = run_dir / train_cfg.grad_norm_log.path
    sh_cfg = train_cfg.state_hash
    flops_tok = transformer_flops_per_token(cfg.model.n_layers, cfg.model.d_model, train_cfg.seq_len, cfg.model.vocab_size)

    if resume_from is None and sh_cfg.at_init and sh_cfg.every_n_steps > 0:
        engine.gather_full_state()
        init_hash = engine.full_state_hash()
        if rank == 0:
            (run_dir / "checkpoints").mkdir(parents=True, exist_ok=True)
            (run_dir / "checkpoints" / "state_hash_init.txt").write_text(init_hash + "\n")
            _append_jsonl(hash_log, {"step": 0, "kind": "init", "consumed_tokens": 0, "state_hash": init_hash})

    tokenizer_hash = ""
    if cfg.run.tokenizer_path and Path(cfg.run.tokenizer_path).is_file():
        from ..data.tokenizer import compute_hash

        tokenizer_hash = compute_hash(cfg.run.tokenizer_path)

    def make_meta() -> CheckpointMeta:
        return CheckpointMeta(consumed_tokens=consumed, step=step, git_sha=git_sha(), config_resolved=resolved_config_json(cfg),
                              tokenizer_hash=tokenizer_hash, container_digest=os.environ.get("CONTAINER_DIGEST", ""),
                              native_source_digests=native_source_digests(),
                              restart_count=restart_count, chained_hash=chained, reduction_mode=cfg.run.reduction_mode, dp_world_size=V,
                              dp_replicate=engine.dp_replicate, dp_shard=engine.dp_shard, tensor_digest=sh_cfg.tensor_digest,
                              rewarm_anchor_tokens=rewarm_anchor, seed=cfg.run.seed, torch_version=torch.__version__,
                              numpy_version=np.__version__, kernel_env={k: v for k, v in os.environ.items() if k.startswith("OTB_")},
                              repop_env={k: v for k, v in os.environ.items() if k.startswith("REPOP_")},
                              windows_emitted=loader.state().windows_emitted, physical_world_size=world,
                              mixed_precision=cfg.run.mixed_precision)

    def global_batch_digest() -> bytes:
        chains = {v: h.local_digest() for v, h in hashers.items()}
        if world > 1:
            objs: list = [None] * world
            dist.all_gather_object(objs, chains, group=engine.host_group)
            chains = {k: v for d in objs for k, v in d.items()}
        return SH.combine_batch_digests([chains[v] for v in range(V)])

    result = {"run_dir": str(run_dir), "hashes": [], "losses": [], "device": str(dev)}
    zero_norm_streak: dict[str, int] = {}
    heartbeat = None
    if world > 1 and cfg.run.heartbeat_timeout_s > 0:
        from ..parallel.heartbeat import Heartbeat

        heartbeat = Heartbeat(rank, world, os.environ.get("MASTER_ADDR", "127.0.0.1"),
                              int(os.environ.get("OTB_HEARTBEAT_PORT") or int(os.environ.get("MASTER_PORT", "29500")) + 1),
                              timeout_s=cfg.run.heartbeat_timeout_s)
    pending_hash: list = []  # at most one (step, consumed, handle, batch digest, advances the chain) whose digests are in flight

    def finish_pending_hash():
        """Fold the state hash whose device digests were started at the end of an earlier step into the chain and the log."""
        nonlocal chained
        if not pending_hash:
            return None
        h_step, h_consumed, handle, bd, due = pending_hash.pop()
        digest = engine.finish_state_hash(handle, chained, bd)
        if due:
            chained = digest
        if rank == 0:
            _append_jsonl(hash_log, {"step": h_step, "consumed_tokens": h_consumed, "state_hash": digest})
        result["hashes"].append((h_step, digest))
        return digest

    try:
        it = iter(loader)
        while consumed < train_cfg.total_tokens and (max_steps is None or step < max_steps):
            t_step = time.perf_counter()
            if heartbeat is not None:
                heartbeat.check()  # a peer that left or died is noticed here, before this step's collectives
            plan, batches = next(it)
            M = plan.microbatches
            if M % V:
                raise RuntimeError("step %d has %d micro-batches, not a multiple of the %d virtual ranks" % (step, M, V))
            accum = M // V
            lr = sched(consumed, train_cfg.total_tokens) * rewarm_factor(consumed, rewarm_anchor, cfg.schedule.rewarm_tokens)
            engine.global_step = step
            engine.zero_grads()
            ces, zs, owners = [], [], []
            batches = list(batches)
            for j, (v, k, windows) in enumerate(batches):
                batch = collate(windows, pin=engine.is_cuda)
                if sh_cfg.include_batch:
                    hashers[v].update(batch)
                ids = batch["input_ids"].to(dev, non_blocking=True)
                labels = batch["labels"].to(dev, non_blocking=True)
                ce, z = engine.forward_backward(hosted.index(v), ids, labels, accum, last=j == len(batches) - 1)
                ces.append(ce.detach())
                zs.append(z.detach())
                owners.append(v)
            finish_pending_hash()  # the previous step's digests ran under this step's forward/backward
            grad_norm = engine.reduce_gradients()
            local_ce = [float(c) for c in ces]
            lead = engine.tp_rank == 0  # the ranks of a tensor-parallel group hold the same values: one of them reports
            # the spike gate looks at virtual rank 0's mean loss ("v0"), on every rank, as the replay does (reference
            # src/pretrain/train/loop.py:977-992, src/pretrain/cli/audit_replay.py:2548-2551)
            sums = deterministic_scalar_sums({"ce": local_ce if lead else [], "z": [float(z) for z in zs] if lead else [],
                                              "v0": [c for c, v in zip(local_ce, owners) if v == 0] if lead else []}, world, engine.host_group)
            (ce_sum, n_mb), (z_sum, _), (v0_sum, v0_n) = sums["ce"], sums["z"], sums["v0"]
            loss_mean = ce_sum / max(n_mb, 1)
            spike_loss = v0_sum / max(v0_n, 1)
            engine.zero_q_gain_grads(step, train_cfg.qk_freeze_q_gains_until_step)
            skipped = spike.should_skip(grad_norm, spike_loss, step)
            clip = engine.clip_coefficient(grad_norm, train_cfg.grad_clip)
            if skipped:
                spike.record_skip(step)
                engine.skip_step()
            else:
                engine.optimizer_step(lr, clip)
                clamp_qk_gains(engine.model, train_cfg.qk_gain_clamp)
            if train_cfg.dead_tensor_assert_steps > 0:
                for name, sos in zip(engine.names, engine.per_tensor_sos):
                    zero_norm_streak[name] = zero_norm_streak.get(name, 0) + 1 if sos == 0.0 else 0
                    if zero_norm_streak[name] >= train_cfg.dead_tensor_assert_steps:
                        raise RuntimeError("parameter %s had an exactly zero gradient for %d consecutive steps" % (name, zero_norm_streak[name]))
            consumed += plan.tokens_this_step
            step += 1

            compute_ms = (time.perf_counter() - t_step) * 1e3  # forward, backward, reduction, clip, update: before hash and checkpoint
            exit_due = _emergency_exit_requested(world, dev, engine.host_group)
            final_step = consumed >= train_cfg.total_tokens or (max_steps is not None and step >= max_steps)
            hash_due = sh_cfg.every_n_steps > 0 and step % sh_cfg.every_n_steps == 0
            ckpt_due = (train_cfg.ckpt_every_steps > 0 and step % train_cfg.ckpt_every_steps == 0) or \
                       (train_cfg.ckpt_every_steps == 0 and train_cfg.ckpt_every_tokens > 0 and
                        consumed // train_cfg.ckpt_every_tokens > (consumed - plan.tokens_this_step) // train_cfg.ckpt_every_tokens)
            step_hash, t_hash = None, 0.0
            if hash_due or ckpt_due or exit_due or final_step:  # a checkpoint is always stamped with its step's hash
                t0 = time.perf_counter()
                bd = global_batch_digest() if sh_cfg.include_batch else None
                pending_hash.append((step, consumed, engine.begin_state_hash(include_grads=sh_cfg.include_grads), bd, hash_due))
                # a checkpoint, an exit or the last step needs the digest now; a plain cadence hash on a GPU is folded in
                # during the next step, after its forward/backward has been queued
                if ckpt_due or exit_due or final_step or not engine.is_cuda:
                    step_hash = finish_pending_hash()
                t_hash = (time.perf_counter() - t0) * 1e3
            t_ckpt = 0.0
            if ckpt_due or exit_due or final_step:
                t0 = time.perf_counter()
                # a cadence checkpoint on GPUs is written in the background from a pinned-host snapshot; the last one of a run
                # (and any on CPU ranks) is committed before going on
                ckpt.save(step, engine, make_meta(), step_hash, loader.state().to_json(), spike.state_dict(),
                          {v: h.local_digest() for v, h in hashers.items()}, wait=exit_due or final_step or not engine.is_cuda)
                t_ckpt = (time.perf_counter() - t0) * 1e3
            wall_ms = (time.perf_counter() - t_step) * 1e3
            result["losses"].append(loss_mean)
            phases = engine.phase_report()  # empty unless PRETRAIN_CUDA_EVENT_TIMING=1
            gl = train_cfg.grad_norm_log
            if gl.every_n_steps > 0 and step % gl.every_n_steps == 0 and gl.weight_stats_every_n_steps > 0 and step % gl.weight_stats_every_n_steps == 0:
                engine.complete_compute_weights()  # the statistics read whole weights (a collective in gather mode, else nothing)
            if rank == 0:
                tps = plan.tokens_this_step / (wall_ms / 1e3)
                z_mean = z_sum / max(n_mb, 1)
                mine_ce = sum(local_ce) / max(len(local_ce), 1)              # this process's micro-batches (the reference's rank-local keys)
                mine_z = sum(float(z) for z in zs) / max(len(zs), 1)
                metrics.log({**phases, "step": step, "consumed_tokens": consumed, "loss": loss_mean, "z_loss": z_mean, "lr": lr,
                             "accum_steps": accum, "loss_ce": mine_ce, "loss_zloss": mine_z, "perplexity": math.exp(min(mine_ce, 700.0)),
                             "loss_ce_global": loss_mean, "loss_zloss_global": z_mean, "perplexity_global": math.exp(min(loss_mean, 700.0)),
                             "grad_norm_pre_clip": grad_norm, "clip_coef": clip, "skipped": skipped,
                             "skipped_steps_total": spike.state.skipped_steps, "tokens_per_sec": tps, "tokens_per_sec_per_gpu": tps / world,
                             "mfu": mfu(tps / world, flops_tok), "step_compute_time_ms": compute_ms, "step_wall_time_ms": wall_ms,
                             "hash_time_ms": t_hash, "ckpt_save_time_ms": t_ckpt, "state_hash": step_hash, "microbatches": M}, step=step)
                gl = train_cfg.grad_norm_log
                if gl.every_n_steps > 0 and step % gl.every_n_steps == 0:
                    from ..obs import grad_norm_log as GN

                    stats = gl.weight_stats_every_n_steps > 0 and step % gl.weight_stats_every_n_steps == 0
                    master = engine.named_weights_for_stats() if stats else None
                    GN.append(gn_log, GN.build_record(step, consumed, engine.names, engine.per_tensor_sos, gl.top_k,
                                                      GN.weight_norms(master) if stats else None, GN.qk_gain_max(master) if stats else None))
            if exit_due:
                log.warning("SIGTERM received: checkpoint written at step %d, exiting", step)
                raise SystemExit(0)
    except Halt as h:
        log.error("halted by the spike protocol: %s", h)
        result["halted"] = str(h)
        finish_pending_hash()
    except BaseException as e:
        if heartbeat is not None and not isinstance(e, SystemExit):
            heartbeat.report_failure("%s: %s" % (type(e).__name__, e))  # the others leave at their next check
        raise
    finally:
        try:
            ckpt.wait()  # a checkpoint still being written in the background is committed (or its error raised) before leaving
        finally:
            if heartbeat is not None:
                heartbeat.close()
            metrics.close()
            engine.close()
    result.update({"step": step, "consumed_tokens": consumed, "chained_hash": chained})
    return result
