"""``pretrain-audit-replay``: re-execute training steps on ONE device and compare the state hash.

The replay hosts all V recorded virtual ranks in a single process (GPU or plain CPU) and runs the very
engine the cluster ran - same kernels or their bit-exact CPU twins, same reduction tree - so an honest
checkpoint chain reproduces digest for digest. Modes:

  --from-init                       rebuild the weights from the seed, check the init hash, optionally continue
  --checkpoint DIR --until-step N   load a checkpoint, replay up to step N
  --expect-hash HEX|FILE            digest to compare with (default: the run's logs/state_hashes.jsonl or the
                                    target checkpoint's state_hash.txt when they can be found)

Prints ``MATCH=True/False``; exit status 1 and ``AUDIT FAILED: state_hash X != Y`` on a mismatch. Result JSON:
{step, consumed_tokens, state_hash, kernels, device, rank0_losses, expected, match, saved_checkpoint?}
(reference src/pretrain/cli/audit_replay.py:1144-1349, 2789-2807).
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import re
import sys
import time
from pathlib import Path

log = logging.getLogger("pretrain.audit")
MAX_AUDIT_WORLD = 64
# The replica fold the reduction kernels implement (parallel/deterministic_reduce.py::tree_reduce_sum), under the tag the
# reference writes for the same combination tree. "binary_blocks_tree" is what earlier versions of this package wrote while
# their kernels used the stride tree, which is the same grouping only while the replica count has at most two set bits.
REPLICATE_REDUCE_ALGOS = {"recursive_doubling"}
LEGACY_REPLICATE_REDUCE_ALGO = "binary_blocks_tree"
_HEX64 = re.compile(r"^[0-9a-fA-F]{64}$")
# kernel-selecting environment a checkpoint may ask the replay to re-apply; anything else is refused
ALLOWED_KERNEL_ENV = {"OTB_EXECUTION_MODE", "OTB_ATTN_BLOCK", "OTB_TENSOR_DIGEST"}
REFUSED_ENV_PREFIXES = ("OTB_LIB", "OTB_CXX", "OTB_REBUILD", "LD_", "PYTHON")


class AuditError(RuntimeError):
    pass


def resolve_expect_hash(value: str | None) -> str | None:
    """A 64-hex digest, or a path to a file whose first token is one."""
    if value is None:
        return None
    if _HEX64.match(value.strip()):
        return value.strip().lower()
    p = Path(value)
    if p.is_file():
        tok = p.read_text().split()
        if tok and _HEX64.match(tok[0]):
            return tok[0].lower()
        raise AuditError("%s does not start with a 64-hex digest" % p)
    raise AuditError("--expect-hash must be a 64-character hex digest or a file containing one, got %r" % value)


def apply_kernel_env(env: dict) -> dict:
    """Re-apply the allow-listed kernel environment recorded in a checkpoint; refuse redirecting keys."""
    applied = {}
    for k, v in (env or {}).items():
        if any(k.startswith(p) for p in REFUSED_ENV_PREFIXES):
            raise AuditError("checkpoint metadata tries to set %s, which could redirect native code; refused" % k)
        if k in ALLOWED_KERNEL_ENV:
            os.environ[k] = str(v)
            applied[k] = str(v)
    return applied


def check_device(device: str) -> None:
    """Refuse a device this process cannot use, before anything is built: ``cuda`` / ``cuda:N`` without a visible GPU (or
    with fewer than N+1), a GPU request on a checkout whose CUDA library was never built, anything that is neither ``cpu``
    nor ``cuda``. (reference src/pretrain/cli/audit_replay.py device guard and audit-kit provenance check)"""
    import torch

    if device == "cpu":
        return
    kind, _, index = device.partition(":")
    if kind != "cuda" or (index and not index.isdigit()):
        raise AuditError("--device %s: this build replays on cpu or cuda[:N]" % device)
    if not torch.cuda.is_available():
        raise AuditError("--device %s requested but no CUDA device is visible" % device)
    if index and int(index) >= torch.cuda.device_count():
        raise AuditError("--device %s requested but only %d CUDA device(s) are visible" % (device, torch.cuda.device_count()))
    from .. import build_native

    if not (build_native.EXT / "libotb_cuda.so").is_file():
        try:
            build_native._nvcc()   # a missing library is built on first use, which needs the compiler
        except RuntimeError:
            raise AuditError("--device %s: this installation has no CUDA kernels (%s is missing and there is no nvcc to build it)"
                             % (device, build_native.EXT / "libotb_cuda.so")) from None


def check_meta_bounds(meta, state_meta=None) -> None:
    """``meta.json`` is untrusted input and the replay's memory and time grow with the recorded world size: implausible
    integers are refused before the model is built. (reference tests/test_audit_meta_bounds.py)"""
    V, S, R = meta.dp_world_size, meta.dp_shard, meta.dp_replicate
    if not all(isinstance(x, int) for x in (V, S, R)) or S < 1 or R < 1 or not (1 <= V <= MAX_AUDIT_WORLD) or S * R != V:
        raise AuditError("recorded topology (world %s = replicate %s x shard %s) is out of bounds (1..%d, factors >= 1, product = world)"
                         % (V, R, S, MAX_AUDIT_WORLD))
    for m in (meta, state_meta):
        if m is not None and (m.step < 0 or m.consumed_tokens < 0):
            raise AuditError("recorded position (step %s, consumed tokens %s) is negative" % (m.step, m.consumed_tokens))


def mismatch_message(got: str, want: str) -> str:
    return "AUDIT FAILED: state_hash %s != %s" % (got, want)


def _find_expected(run_dir: Path | None, step: int) -> str | None:
    if run_dir is None:
        return None
    logf = run_dir / "logs" / "state_hashes.jsonl"
    if logf.is_file():
        for line in logf.read_text().splitlines():
            row = json.loads(line)
            if row.get("step") == step and row.get("kind") != "init":
                return row["state_hash"]
    p = run_dir / "checkpoints" / ("step_%09d" % step) / "state_hash.txt"
    return p.read_text().strip() if p.is_file() else None


def memlog(tag: str, device: str = "cpu") -> dict | None:
    """With PRETRAIN_AUDIT_MEMLOG=1: log (and return) the process's resident set and, on a GPU, the allocator's current,
    peak and reserved bytes at the named point of the replay (reference src/pretrain/cli/audit_replay.py:241-294)."""
    if os.environ.get("PRETRAIN_AUDIT_MEMLOG") != "1":
        return None
    import resource

    rec = {"at": tag, "rss_peak_gib": round(resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 2 ** 20, 3)}
    try:
        with open("/proc/self/statm") as fh:
            rec["rss_gib"] = round(int(fh.read().split()[1]) * os.sysconf("SC_PAGE_SIZE") / 2 ** 30, 3)
    except OSError:
        pass
    if device.startswith("cuda"):
        import torch

        rec.update(cuda_alloc_gib=round(torch.cuda.memory_allocated() / 2 ** 30, 3), cuda_peak_gib=round(torch.cuda.max_memory_allocated() / 2 ** 30, 3),
                   cuda_reserved_gib=round(torch.cuda.memory_reserved() / 2 ** 30, 3))
    log.info("memlog %s", json.dumps(rec))
    return rec


def memory_plan(n_params: int, V: int, R: int, mixed: bool, activation_bytes: int, free_bytes: int | None, reserve_bytes: int,
                offload_grads: bool, offload_optimizer: bool) -> dict:
    """Decide the replay's memory plan before the engine is built. Resident state is 16 bytes per parameter (fp32 master,
    two moments, reduced gradient) plus 2 for bf16 compute weights, plus one 4-byte gradient buffer per virtual rank.
    When that, the activations of one micro-batch and the reserve do not fit into ``free_bytes``, folded gradients are
    switched on first (V buffers -> R + 1), then the moment offload (-8 bytes per parameter). Explicit requests are kept.
    ``free_bytes`` None (unknown) leaves the requests as they are.
    (reference src/pretrain/cli/audit_replay.py:508-711: _plan_optimizer_offload / _plan_master_offload / _plan_grad_offload)"""
    def need(fold: bool, off_opt: bool) -> int:
        per = 16 + (2 if mixed else 0) - (8 if off_opt else 0)
        bufs = (R + 1) if fold else V
        return n_params * (per + 4 * bufs) + activation_bytes + reserve_bytes

    plan = {"offload_grads": bool(offload_grads), "offload_optimizer": bool(offload_optimizer), "auto": [], "free_bytes": free_bytes}
    if free_bytes is not None:
        if need(plan["offload_grads"], plan["offload_optimizer"]) > free_bytes and not plan["offload_grads"] and V > R + 1:
            plan["offload_grads"] = True
            plan["auto"].append("offload_grads")
        if need(plan["offload_grads"], plan["offload_optimizer"]) > free_bytes and not plan["offload_optimizer"]:
            plan["offload_optimizer"] = True
            plan["auto"].append("offload_optimizer")
    plan["need_bytes"] = need(plan["offload_grads"], plan["offload_optimizer"])
    plan["fits"] = free_bytes is None or plan["need_bytes"] <= free_bytes
    return plan


def _free_bytes(device: str) -> int | None:
    try:
        if device.startswith("cuda"):
            import torch

            return int(torch.cuda.mem_get_info()[0])
        import psutil

        return int(psutil.virtual_memory().available)
    except Exception:  # noqa: BLE001 - an unknown amount of memory only disables the automatic plan
        return None


def run_provenance_digests() -> dict:
    from ..utils.git import native_source_digests

    return native_source_digests()


def audit_replay(checkpoint: str | None = None, *, config_name: str | None = None, overrides: list[str] | None = None,
                 data_root: str | None = None, device: str = "cpu", cpu_threads: str | None = None, from_init: bool = False,
                 descriptor_checkpoint: str | None = None, until_step: int | None = None, expect_hash: str | None = None,
                 save_checkpoint_dir: str | None = None, loss_log: str | None = None, run_dir: str | None = None,
                 offload_optimizer: bool = False, offload_master: bool = False, offload_grads: bool = False,
                 fold_spill_dir: str | None = None, no_fold_spill: bool = False, optimizer_offload_dir: str | None = None,
                 master_offload_dir: str | None = None, **_ignored) -> dict:
    import numpy as np
    import torch

    from ..config import load_config, parse_config_resolved
    from ..data.global_stream import GlobalStreamState
    from ..data.loader import build_global_loader, collate
    from ..optim.schedules import build_schedule, rewarm_factor
    from ..ops import native
    from ..train import state_hash as SH
    from ..train.checkpoint import CheckpointMeta, Checkpointer, resolved_config_json
    from ..train.engine import TrainEngine
    from ..train.spike_protocol import Halt, SpikeProtocol
    from ..train.qk_gain_control import clamp_qk_gains
    from .cpu_threads import configure_cpu_threads

    expected = resolve_expect_hash(expect_hash)
    if device == "cpu":
        configure_cpu_threads(cpu_threads or "auto")
    check_device(device)
    if not from_init and checkpoint is None:
        raise AuditError("either --checkpoint or --from-init (with --config-name or --descriptor-checkpoint) is required")

    # Two roles of a checkpoint's metadata. The DESCRIPTOR says how the interval was trained (configuration, topology,
    # kernel environment, re-warm anchor): it comes from --descriptor-checkpoint when given, else from --checkpoint. The
    # POSITION (step, consumed tokens, chained hash, stream state) always comes from --checkpoint, whose state is loaded.
    # A resume boundary is audited with the old run's last checkpoint as the state and the resumed run's first checkpoint
    # as the descriptor. (reference src/pretrain/cli/audit_replay.py:1166-1186)
    meta = None
    src = descriptor_checkpoint or checkpoint
    state_meta = Checkpointer.read_meta(checkpoint) if (checkpoint is not None and not from_init) else None
    if src is not None:
        meta = Checkpointer.read_meta(src)
        apply_kernel_env(meta.kernel_env)
        if run_dir is None:
            run_dir = str(Path(src).resolve().parent.parent)
        if state_meta is not None and descriptor_checkpoint is not None and state_meta.seed != meta.seed:
            raise AuditError("--descriptor-checkpoint was trained with seed %s, --checkpoint with seed %s: not the same run lineage"
                             % (meta.seed, state_meta.seed))
    if meta is not None and meta.config_resolved and config_name is None:
        cfg = parse_config_resolved(meta.config_resolved)
    elif config_name is not None:
        cfg = load_config(config_name, overrides or [])
    else:
        raise AuditError("no configuration: the checkpoint has none embedded and --config-name was not given")
    if cfg.run.reduction_mode != "deterministic_allgather":
        raise AuditError("run.reduction_mode=%s is not auditable (only deterministic_allgather pins the reduction order)" % cfg.run.reduction_mode)
    if cfg.run.parallel == "ddp":
        raise AuditError("run.parallel=ddp is not auditable (library all-reduce, reduction order not pinned)")
    if meta is not None:
        check_meta_bounds(meta, state_meta)
        V, S, R = meta.dp_world_size, meta.dp_shard, meta.dp_replicate
        if meta.clip_algo != "global" or meta.grad_norm_algo != "deterministic_per_tensor_sos_v1":
            raise AuditError("unsupported clip / norm algorithm in checkpoint metadata")
        legacy_ok = meta.replicate_reduce_algo == LEGACY_REPLICATE_REDUCE_ALGO and bin(max(meta.dp_replicate, 0)).count("1") <= 2
        if meta.replicate_reduce_algo not in REPLICATE_REDUCE_ALGOS and not legacy_ok:
            raise AuditError("this replay knows the replica orders %s; the checkpoint was trained with replicate_reduce_algo=%r"
                             % (sorted(REPLICATE_REDUCE_ALGOS), meta.replicate_reduce_algo))
        cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size = V, S, R
    elif cfg.run.virtual_dp_size == 0:
        raise AuditError("--from-init with --config-name needs run.virtual_dp_size (the topology to emulate)")

    if until_step is not None and state_meta is not None and until_step <= state_meta.step:
        raise AuditError("--until-step %d is not beyond the starting step %d" % (until_step, state_meta.step))  # before anything is built

    cfg.run.tp_size = 1  # a tensor-parallel run is replayed unsplit: the split never changes a bit
    # --offload-grads: one work buffer plus one partial per replica instead of one gradient buffer per virtual rank
    # (each finished virtual rank is folded into its replica's partial, ascending shard order); --fold-spill-dir puts
    # the finished partials on disk with a digest that is checked when they are read back
    from ..obs.metrics import count_parameters

    m = cfg.model
    mb_tokens = cfg.train.micro_batch_size * cfg.train.seq_len
    act = mb_tokens * (m.n_layers * 30 * m.d_model * (2 if cfg.run.mixed_precision else 4) // 2 + 6 * m.vocab_size)
    plan = memory_plan(count_parameters(m), cfg.run.virtual_dp_size, max(1, cfg.run.dp_replicate_size), bool(cfg.run.mixed_precision), act,
                       _free_bytes(device), int(float(os.environ.get("PRETRAIN_AUDIT_MEM_RESERVE_GB", "4")) * 2 ** 30),
                       offload_grads, offload_optimizer)
    init_only = from_init and until_step in (None, 0)
    if init_only:
        # an init audit never runs a step: gradient buffers and moments stay untouched zero pages, no activations exist, and
        # moments kept in files would only make the full hash read them back. The plan is for replays that train.
        offload_grads = True   # one work buffer instead of one per virtual rank; nothing is ever written to it
    else:
        for what in plan["auto"]:
            log.warning("memory plan: %s AUTO-ENABLED - %.1f GiB free is less than the default plan needs; pass the flag to make it explicit",
                        what, plan["free_bytes"] / 2 ** 30)
        if not plan["fits"]:
            log.warning("memory plan: about %.1f GiB needed, %.1f GiB free - the replay may run out of memory", plan["need_bytes"] / 2 ** 30,
                        plan["free_bytes"] / 2 ** 30)
        offload_grads, offload_optimizer = plan["offload_grads"], plan["offload_optimizer"]
    spill = None if (no_fold_spill or not offload_grads) else fold_spill_dir
    # --offload-optimizer / --offload-master: moments / fp32 master weights live in files between steps
    engine = TrainEngine(cfg, device, 0, 1, init=from_init or checkpoint is None, fold_gradients=offload_grads, fold_spill_dir=spill,
                         offload_optimizer=offload_optimizer, optimizer_offload_dir=optimizer_offload_dir,
                         offload_master=offload_master, master_offload_dir=master_offload_dir)
    if engine.master_offload_inert:
        log.warning("--offload-master changes nothing on a GPU: the fp32 master weights stay resident")
    if meta is not None and meta.native_source_digests:
        here = run_provenance_digests()
        differing = sorted(k for k, v in meta.native_source_digests.items() if k in here and here[k] != v)
        if differing:
            log.warning("native sources differ from the build that wrote the checkpoint (%s): a mismatch may come from the build, "
                        "not from the run", ", ".join(differing))
    memlog("engine built", device)
    V = engine.V
    run_path = Path(run_dir) if run_dir else None
    from ..utils.git import run_provenance

    result: dict = {"device": device, "kernels": native.loaded_libraries(), "build": run_provenance(), "rank0_losses": [], "expected": expected,
                    "match": None}
    step, consumed, chained, stream_state = 0, 0, None, None
    hashers = {v: SH.RunningBatchHasher() for v in range(V)}
    spike = SpikeProtocol.from_config(cfg.train.spike)
    rewarm_anchor = None

    if from_init:
        init_hash = engine.full_state_hash()
        want = expected if (until_step in (None, 0)) else None
        if want is None and run_path is not None and (run_path / "checkpoints" / "state_hash_init.txt").is_file():
            want = (run_path / "checkpoints" / "state_hash_init.txt").read_text().strip()
        result.update({"init_hash": init_hash, "init_expected": want, "init_match": (init_hash == want) if want else None})
        if want and init_hash != want:
            result.update({"step": 0, "consumed_tokens": 0, "state_hash": init_hash, "expected": want, "match": False})
            return result
        if until_step in (None, 0):
            result.update({"step": 0, "consumed_tokens": 0, "state_hash": init_hash, "expected": want, "match": (init_hash == want) if want else None})
            return result
    else:
        ck = Checkpointer(Path(checkpoint).parent.parent)
        side = ck.load(checkpoint, engine)
        step, consumed, chained = state_meta.step, state_meta.consumed_tokens, state_meta.chained_hash
        stream_state = GlobalStreamState.from_json(side["global_stream"]) if side["global_stream"] else None
        hashers = {v: SH.RunningBatchHasher(side["batch_chains"][v]) for v in range(V)}
        spike.load_state_dict(side["spike_protocol"])
        rewarm_anchor = meta.rewarm_anchor_tokens if descriptor_checkpoint is not None else state_meta.rewarm_anchor_tokens
    if until_step is None:
        # default span: one checkpoint interval of the recipe (steps, or tokens when the recipe clocks checkpoints by tokens)
        from ..train.batch_schedule import default_interval_end

        until_step = default_interval_end(step, consumed, cfg.train)
    if until_step <= step:
        raise AuditError("--until-step %d is not beyond the starting step %d" % (until_step, step))

    tr, sh_cfg = cfg.train, cfg.train.state_hash
    sched = build_schedule(cfg.schedule, tr, cfg.optim)
    loader = build_global_loader(cfg, list(range(V)), V, state=stream_state, consumed_tokens=consumed, start_step=step, data_root=data_root)
    dev = torch.device(device)
    # PRETRAIN_AUDIT_EMPTY_CACHE_PER_MB=1: hand cached allocator blocks back after every micro-batch (tight GPUs)
    empty_cache_per_mb = os.environ.get("PRETRAIN_AUDIT_EMPTY_CACHE_PER_MB") == "1" and device.startswith("cuda")
    last_hash = None
    loss_rows = []
    t_start = time.time()
    for plan, batches in loader:
        if step >= until_step:
            break
        accum = plan.microbatches // V
        lr = sched(consumed, tr.total_tokens) * rewarm_factor(consumed, rewarm_anchor, cfg.schedule.rewarm_tokens)
        engine.global_step = step
        engine.zero_grads()
        ces = []
        if engine.fold:
            # the loader yields micro-batches in global order (owner m mod V), which interleaves the virtual ranks; the
            # folded mode has one work buffer, so it runs virtual rank by virtual rank, each rank's micro-batches ascending
            batches = sorted(batches, key=lambda b: (b[0], b[1]))
        halted = None
        batches = list(batches)
        for j, (v, k, windows) in enumerate(batches):
            batch = collate(windows)
            if sh_cfg.include_batch:
                hashers[v].update(batch)
            ce, z = engine.forward_backward(v, batch["input_ids"].to(dev), batch["labels"].to(dev), accum, last=j == len(batches) - 1)
            ces.append((v, k, float(ce.detach())))
            if empty_cache_per_mb:
                torch.cuda.empty_cache()
            if engine.fold and k == accum - 1:
                engine.fold_virtual_rank(v)  # all of v's micro-batches are in the work buffer
        memlog("step %d: after forward/backward" % (step + 1), device)
        grad_norm = engine.reduce_gradients()
        total = 0.0
        for _, _, c in ces:
            total += c
        loss_mean = total / max(len(ces), 1)
        v0 = [c for v, _, c in sorted(ces, key=lambda t: (t[0], t[1])) if v == 0]
        v0_sum = 0.0
        for c in v0:
            v0_sum += c
        spike_loss = v0_sum / max(len(v0), 1)  # virtual rank 0's mean loss, as in the training loop
        engine.zero_q_gain_grads(step, tr.qk_freeze_q_gains_until_step)  # mirrors train/loop.py
        if spike.should_skip(grad_norm, spike_loss, step):
            try:
                spike.record_skip(step)
            except Halt as h:
                halted = str(h)  # the step's hash is still recorded below, then the replay ends (as the run did)
            engine.skip_step()
        else:
            engine.optimizer_step(lr, engine.clip_coefficient(grad_norm, tr.grad_clip))
            clamp_qk_gains(engine.model, tr.qk_gain_clamp)
        consumed += plan.tokens_this_step
        step += 1
        r0 = [c for v, _, c in ces if v == 0]
        result["rank0_losses"].extend(r0)
        loss_rows.append({"step": step, "rank0_losses": r0, "loss": loss_mean, "grad_norm": grad_norm})
        hash_due = sh_cfg.every_n_steps > 0 and step % sh_cfg.every_n_steps == 0
        ckpt_due = tr.ckpt_every_steps > 0 and step % tr.ckpt_every_steps == 0
        if hash_due or ckpt_due or step == until_step:
            bd = SH.combine_batch_digests([hashers[v].local_digest() for v in range(V)]) if sh_cfg.include_batch else None
            last_hash = engine.sharded_state_hash(chained, bd, include_grads=sh_cfg.include_grads, tensor_digest=sh_cfg.tensor_digest)
            if hash_due:
                chained = last_hash
        engine.release_state()
        memlog("step %d: end" % step, device)
        phases = engine.phase_report()  # PRETRAIN_CUDA_EVENT_TIMING=1
        if phases:
            log.info("step %d phases %s", step, json.dumps({k: round(v, 3) for k, v in phases.items()}))
        log.info("replayed step %d loss %.6f grad_norm %.6f", step, loss_mean, grad_norm)
        if halted is not None:
            if last_hash is None or not (hash_due or ckpt_due or step == until_step):
                bd = SH.combine_batch_digests([hashers[v].local_digest() for v in range(V)]) if sh_cfg.include_batch else None
                last_hash = engine.sharded_state_hash(chained, bd, include_grads=sh_cfg.include_grads, tensor_digest=sh_cfg.tensor_digest)
            result["halted"] = halted
            log.error("the spike protocol halted the run at step %d: %s", step, halted)
            break
    result["seconds_per_step"] = (time.time() - t_start) / max(len(loss_rows), 1)
    if torch.cuda.is_available() and device.startswith("cuda"):
        result["peak_memory_bytes"] = int(torch.cuda.max_memory_allocated())
    if expected is None:
        expected = _find_expected(run_path, step)
    result.update({"step": step, "consumed_tokens": consumed, "state_hash": last_hash, "expected": expected,
                   "match": (last_hash == expected) if expected else None})
    if loss_log:
        Path(loss_log).write_text("\n".join(json.dumps(r) for r in loss_rows) + "\n")
    diff_against = os.environ.get("PRETRAIN_AUDIT_DIFF_CKPT") or os.environ.get("REPOP_AUDIT_DIFF_CKPT")
    if diff_against:
        result["diff"] = diff_against_checkpoint(engine, diff_against)
    if save_checkpoint_dir:
        ck = Checkpointer(save_checkpoint_dir)
        m = CheckpointMeta(consumed_tokens=consumed, step=step, config_resolved=resolved_config_json(cfg), chained_hash=chained,
                           reduction_mode=cfg.run.reduction_mode, dp_world_size=V, dp_replicate=engine.dp_replicate, dp_shard=engine.dp_shard,
                           tensor_digest=sh_cfg.tensor_digest, seed=cfg.run.seed, torch_version=torch.__version__, numpy_version=np.__version__,
                           windows_emitted=loader.state().windows_emitted, mixed_precision=cfg.run.mixed_precision)
        d = ck.save(step, engine, m, last_hash, loader.state().to_json(), spike.state_dict(), {v: h.local_digest() for v, h in hashers.items()})
        from .verify_handoff import write_gradient_sidecar

        write_gradient_sidecar(d, engine.named_grads())
        result["saved_checkpoint"] = str(d)
    engine.close()
    return result


def diff_against_checkpoint(engine, checkpoint: str, top: int = 15) -> dict:
    """Where a replay and a checkpoint part ways, tensor by tensor (a diagnostic for a hash mismatch; it changes nothing of
    the replay): the largest absolute difference of every master weight and of both moments between the replayed state and
    the checkpoint named by PRETRAIN_AUDIT_DIFF_CKPT (the reference's REPOP_AUDIT_DIFF_CKPT is read too,
    src/pretrain/cli/audit_replay.py:2725-2760). Returns {"tensors", "differing", "top": [[max |delta|, kind, name], ...]}."""
    import torch

    from ..train.checkpoint import optimizer_state_names
    from .dcp_safetensors import read_dcp

    state = read_dcp(Path(checkpoint) / "dcp")
    names = optimizer_state_names(checkpoint)          # optimizer-state key (an index as a string) -> parameter name
    rows = []
    mine = dict(engine.named_master())
    for name, theirs in (state.get("model") or {}).items():
        if name in mine:
            rows.append((float((mine[name].detach().float().cpu() - theirs.float()).abs().max()), "param", name))
    moments = engine.optimizer_state()
    for key, st in ((state.get("optim") or {}).get("state") or {}).items():
        name = names.get(str(key), str(key))
        if name not in moments:
            continue
        for kind in ("exp_avg", "exp_avg_sq"):
            if kind in st and torch.is_tensor(st[kind]):
                rows.append((float((moments[name][kind].detach().float().cpu() - st[kind].float()).abs().max()), "optim." + kind, name))
    rows.sort(key=lambda r: -r[0])
    differing = sum(1 for r in rows if r[0] > 0)
    log.info("DIFF against %s: %d of %d tensors differ; largest differences:", checkpoint, differing, len(rows))
    for d, kind, name in rows[:top]:
        log.info("  max|delta|=%.6e  %s  %s", d, kind, name)
    return {"against": str(checkpoint), "tensors": len(rows), "differing": differing, "top": [[d, kind, name] for d, kind, name in rows[:top]]}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pretrain-audit-replay", description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint")
    ap.add_argument("--config-name")
    ap.add_argument("--data-root")
    ap.add_argument("--gcs-root")
    ap.add_argument("--fetch-dest")
    ap.add_argument("--device", default="cpu", choices=["cuda", "cpu", "mps"])
    ap.add_argument("--cpu-threads", default=None)
    ap.add_argument("--from-init", action="store_true")
    ap.add_argument("--descriptor-checkpoint")
    ap.add_argument("--until-step", type=int)
    ap.add_argument("--expect-hash")
    ap.add_argument("--fold-spill-dir")
    ap.add_argument("--no-fold-spill", action="store_true")
    ap.add_argument("--offload-optimizer", action="store_true")
    ap.add_argument("--optimizer-offload-dir")
    ap.add_argument("--offload-master", action="store_true")
    ap.add_argument("--offload-grads", action="store_true")
    ap.add_argument("--master-offload-dir")
    ap.add_argument("--save-checkpoint-dir")
    ap.add_argument("--loss-log")
    ap.add_argument("--run-dir")
    ap.add_argument("overrides", nargs="*")
    return ap


def main(argv: list[str] | None = None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(message)s")
    from ._args import parse_with_overrides

    a = parse_with_overrides(build_parser(), argv)
    if a.device == "mps":
        print("AUDIT ERROR: Apple Metal/MPS is unavailable on this platform; use --device cuda or cpu", file=sys.stderr)
        return 2
    if a.gcs_root or a.fetch_dest:
        from ..data.fetch_interval import fetch_audit_interval

        if a.checkpoint and a.gcs_root:
            a.data_root = fetch_audit_interval(a.checkpoint, a.gcs_root, a.fetch_dest or "audit_data", until_step=a.until_step,
                                               config_name=a.config_name, from_init=a.from_init).data_root
    try:
        res = audit_replay(a.checkpoint, config_name=a.config_name, overrides=a.overrides, data_root=a.data_root, device=a.device,
                           cpu_threads=a.cpu_threads, from_init=a.from_init, descriptor_checkpoint=a.descriptor_checkpoint,
                           until_step=a.until_step, expect_hash=a.expect_hash, save_checkpoint_dir=a.save_checkpoint_dir,
                           loss_log=a.loss_log, run_dir=a.run_dir, offload_optimizer=a.offload_optimizer, offload_master=a.offload_master,
                           offload_grads=a.offload_grads, fold_spill_dir=a.fold_spill_dir, no_fold_spill=a.no_fold_spill,
                           optimizer_offload_dir=a.optimizer_offload_dir, master_offload_dir=a.master_offload_dir)
    except AuditError as e:
        print("AUDIT ERROR: %s" % e, file=sys.stderr)
        return 2
    print(json.dumps(res, indent=1, default=str))
    log.info("MATCH=%s", res["match"])
    print("MATCH=%s" % res["match"])
    if res["match"] is False:
        print(mismatch_message(res["state_hash"], res["expected"]), file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
