"""``pretrain-audit-verify-handoff``: check a downloaded hand-off checkpoint against the hash the run PUBLISHED, from disk
alone - no forward pass, no backward pass, no data.

A hand-off is a checkpoint with ``gradients.safetensors`` beside it: the chained state hash folds in the target step's
post-clip gradients, which an ordinary checkpoint does not carry. The verifier loads weights and moments from ``dcp/``,
reattaches the gradients bit for bit, rebuilds the batch term from every virtual rank's ``batch_hasher.rank_<v>.bin`` and
the previous link from ``--prev-hash``, recomputes the sharded hash in the recorded topology and compares it with
``--expect-hash``. Both digests are literals that the caller takes from the run's published ``logs/state_hashes.jsonl``:
the artifact's own ``state_hash.txt`` is never the target (whoever can write the tensors can write that file); it is read
only to refuse early when the author's claim already disagrees with the published value.

A match covers what the hash covers - weights, moments, parameter groups, the step's gradients, the batch chain. RNG state,
the stream cursor, spike state and the descriptor keys of ``meta.json`` are outside it.

Every refusal is a ``HandoffError``: a reason not to spend a replay on the artifact, never a "probably fine".
(reference src/pretrain/cli/verify_handoff.py:68-443)"""
from __future__ import annotations

import argparse
import json
import logging
import re
import sys
from pathlib import Path

GRAD_FILE = "gradients.safetensors"
GRAD_FORMAT = "pretrain-audit-gradients"
GRAD_VERSION = "1"
_DIGEST = re.compile(r"^[0-9a-fA-F]{64}$")
log = logging.getLogger("pretrain.audit.verify")


class HandoffError(Exception):
    """The hand-off cannot be verified."""


def write_gradient_sidecar(ckpt_dir, named_grads: dict) -> Path:
    """``gradients.safetensors``: one tensor per parameter that has a gradient; the names of those that have none travel
    in the header, so that an absent entry can never be read as "no gradient"."""
    from safetensors.torch import save_file

    tensors, none_names = {}, []
    for name, g in named_grads.items():
        if g is None:
            none_names.append(name)
        else:
            tensors[name] = g.detach().to("cpu").contiguous().clone()
    p = Path(ckpt_dir) / GRAD_FILE
    save_file(tensors, str(p), metadata={"format": GRAD_FORMAT, "format_version": GRAD_VERSION, "none_grad_names": json.dumps(sorted(none_names))})
    return p


def read_gradient_sidecar(ckpt_dir) -> dict:
    """{name: tensor | None} of a hand-off's gradient file; every malformed form is a ``HandoffError``."""
    import safetensors

    p = Path(ckpt_dir) / GRAD_FILE
    if not p.is_file():
        raise HandoffError("%s is missing: the published hash folds in the step's gradients, so without them it cannot be rebuilt - and "
                           "an absent file is never read as 'every gradient was None'. Not an audit hand-off." % p)
    try:
        with safetensors.safe_open(str(p), framework="pt", device="cpu") as f:
            md = f.metadata() or {}
            if md.get("format") != GRAD_FORMAT or md.get("format_version") != GRAD_VERSION:
                raise HandoffError("%s: unsupported gradient file format %r / version %r" % (p, md.get("format"), md.get("format_version")))
            none_names = json.loads(md["none_grad_names"])
            if not isinstance(none_names, list) or not all(isinstance(n, str) for n in none_names):
                raise HandoffError("%s: none_grad_names must be a list of strings" % p)
            tensors = {k: f.get_tensor(k) for k in f.keys()}
    except (OSError, ValueError, KeyError, safetensors.SafetensorError) as e:
        raise HandoffError("%s: invalid gradient file: %s: %s" % (p, type(e).__name__, e)) from e
    if len(set(none_names)) != len(none_names):
        raise HandoffError("%s lists a name twice in none_grad_names" % p)
    both = sorted(set(tensors) & set(none_names))
    if both:
        raise HandoffError("%s lists %s both as a tensor and as a parameter without gradient" % (p, both[:4]))
    out: dict = dict(tensors)
    out.update({n: None for n in none_names})
    return out


def attach_gradients(engine, grads: dict, where: str = GRAD_FILE) -> int:
    """Copy a hand-off's gradients into the engine's reduced-gradient buffer, bits unchanged. The file has to account for
    every parameter exactly once (a tensor, or a name in ``none_grad_names``) with the parameter's shape and fp32 storage;
    a file written for another model is refused here instead of producing an unexplained mismatch. Returns the number of
    tensors attached. (role of the reference's src/pretrain/cli/verify_handoff.py:73-137)"""
    import torch

    lay = engine.layout
    shapes = {n: tuple(lay.shapes[i]) for i, n in enumerate(engine.names)}
    extra = sorted(set(grads) - set(shapes))
    if extra:
        raise HandoffError("%s carries entries for parameters this model does not have: %s" % (where, extra[:4]))
    missing = sorted(set(shapes) - set(grads))
    if missing:
        raise HandoffError("%s accounts for no gradient at all for %s - neither a tensor nor a None entry: incomplete" % (where, missing[:4]))
    for n, g in grads.items():
        if g is not None and (g.dtype != torch.float32 or tuple(g.shape) != shapes[n]):
            raise HandoffError("%s: gradient of %s is %s %s, the parameter's gradient is torch.float32 %s"
                               % (where, n, g.dtype, tuple(g.shape), shapes[n]))
    attached = 0
    engine.grad_red.zero_()
    for i, n in enumerate(engine.names):
        if grads[n] is not None:
            lay.view(engine.grad_red, i).copy_(grads[n])
            attached += 1
    return attached


def read_batch_digest(ckpt_dir, dp_world_size: int) -> bytes:
    """The run's global batch digest from the per-rank chains, combined in rank order. Every rank's file is needed: fewer
    files would hash another schema and report a divergence that is none."""
    from ..train.state_hash import combine_batch_digests

    chains = []
    for v in range(dp_world_size):
        p = Path(ckpt_dir) / ("batch_hasher.rank_%d.bin" % v)
        if not p.is_file():
            raise HandoffError("%s is missing: this hand-off declares dp_world_size=%d, and the state hash folds in the digest of all "
                               "%d per-rank batch chains" % (p, dp_world_size, dp_world_size))
        b = p.read_bytes()
        if len(b) != 32:
            raise HandoffError("%s holds %d bytes; a batch chain is a 32-byte digest" % (p, len(b)))
        chains.append(b)
    try:
        return combine_batch_digests(chains)
    except ValueError as e:
        raise HandoffError("%s: invalid batch chains: %s" % (ckpt_dir, e)) from e


def verify_loaded_state(engine, checkpoint, *, expect_hash: str, prev_hash: str, include_grads: bool, include_batch: bool,
                        tensor_digest: str = "raw") -> dict:
    """The gate over an engine whose weights and moments are already loaded: attach the gradients, rebuild the batch term,
    recompute, compare. The gradients are cleared before returning (a continuation must not inherit them)."""
    checkpoint = Path(checkpoint)
    attached = None
    try:
        if include_grads:
            attached = attach_gradients(engine, read_gradient_sidecar(checkpoint), str(checkpoint / GRAD_FILE))
        bd = read_batch_digest(checkpoint, engine.V) if include_batch else None
        got = engine.sharded_state_hash(prev_hash, bd, include_grads=include_grads, tensor_digest=tensor_digest)
    finally:
        engine.grad_red.zero_()
    return {"verified": got == expect_hash, "reconstructed_hash": got, "expected_hash": expect_hash, "prev_hash": prev_hash,
            "dp_world_size": engine.V, "dp_shard": engine.dp_shard, "include_grads": include_grads, "include_batch": include_batch,
            "gradients_attached": attached}


def read_descriptor(checkpoint: Path) -> dict:
    meta_path = checkpoint / "meta.json"
    if not meta_path.is_file():
        raise HandoffError("%s is missing: not a complete hand-off checkpoint, its topology and hash cadence are unknown" % meta_path)
    if not (checkpoint / "_COMPLETE").is_file():
        raise HandoffError("%s carries no _COMPLETE marker: the writer never finished it, or the download is partial" % checkpoint)
    try:
        meta = json.loads(meta_path.read_text())
    except (OSError, ValueError) as e:
        raise HandoffError("%s is not readable JSON: %s" % (meta_path, e)) from e
    if not isinstance(meta, dict):
        raise HandoffError("%s must hold a JSON object" % meta_path)
    if type(meta.get("step")) is not int or meta["step"] <= 0:
        raise HandoffError("%s: step must be a positive integer" % meta_path)
    return meta


def verify_handoff(checkpoint, *, expect_hash: str, prev_hash: str, config_name: str | None = None, device: str = "cpu") -> dict:
    """Rebuild the hand-off's published hash and compare. ``expect_hash``: the run's published hash of the checkpoint's OWN
    step; ``prev_hash``: the published hash of the previous HASHED step (with a cadence of N that is N steps back)."""
    import torch

    from ..config import load_config, parse_config_resolved
    from ..train.checkpoint import Checkpointer, CheckpointMeta
    from .audit_replay import MAX_AUDIT_WORLD, AuditError, apply_kernel_env

    checkpoint = Path(checkpoint)
    for flag, value in (("--expect-hash", expect_hash), ("--prev-hash", prev_hash)):
        if not isinstance(value, str) or not _DIGEST.match(value.strip()):
            raise HandoffError("%s must be a full literal hex digest from the published log, not a file path or a truncated digest" % flag)
    expect_hash, prev_hash = expect_hash.strip().lower(), prev_hash.strip().lower()
    raw = read_descriptor(checkpoint)
    meta = CheckpointMeta.from_json(json.dumps(raw))
    cfg = load_config(config_name) if config_name else parse_config_resolved(meta.config_resolved)
    # The cadence and content switches come from the artifact's own metadata, which the hash does not authenticate. That is
    # safe because they are inputs of the digest: an author who understates dp_shard or turns the gradients off computes
    # another value and fails the comparison.
    sh, step = cfg.train.state_hash, meta.step
    if sh.every_n_steps <= 0:
        raise HandoffError("the run that wrote this hand-off did not hash its state (state_hash.every_n_steps is 0): there is no "
                           "published commitment to verify it against")
    if step % sh.every_n_steps != 0:
        raise HandoffError("step %d is off the run's hash cadence (every %d steps): the published log holds no hash for it, and such a "
                           "checkpoint stamps a side-link that its metadata does not chain from. Unsupported." % (step, sh.every_n_steps))
    stamped = checkpoint / "state_hash.txt"
    claimed = stamped.read_text().strip().lower() if stamped.is_file() else None
    if claimed is not None and claimed != str(raw.get("chained_hash") or "").lower():
        raise HandoffError("%s (%s...) disagrees with the running chain in meta.json (%s...): not a plain hash-due checkpoint; refusing "
                           "to guess which value the published chain continues from" % (stamped, claimed[:16], str(raw.get("chained_hash"))[:16]))
    if claimed is not None and claimed != expect_hash:
        raise HandoffError("this hand-off claims another state than the run published for step %d:\n    the artifact says  %s\n"
                           "    the run published  %s\nThe published log is authoritative." % (step, claimed, expect_hash))
    V, R, S = raw.get("dp_world_size") or 1, raw.get("dp_replicate") or 1, raw.get("dp_shard") or (raw.get("dp_world_size") or 1)
    if not all(type(x) is int for x in (V, R, S)) or not (1 <= V <= MAX_AUDIT_WORLD) or S < 1 or R < 1:
        raise HandoffError("hand-off declares an implausible topology (dp_world_size=%r, dp_replicate=%r, dp_shard=%r); the cap is %d"
                           % (V, R, S, MAX_AUDIT_WORLD))
    if R * S != V:
        raise HandoffError("hand-off topology is inconsistent: dp_replicate(%d) * dp_shard(%d) != dp_world_size(%d)" % (R, S, V))
    # files the digest needs: their absence is a refusal that costs nothing, so it comes before the model is built
    if sh.include_batch:
        read_batch_digest(checkpoint, V)
    if sh.include_grads and not (checkpoint / GRAD_FILE).is_file():
        read_gradient_sidecar(checkpoint)
    dev = torch.device(device)
    if dev.type == "cuda" and not torch.cuda.is_available():
        raise HandoffError("CUDA is unavailable; use --device cpu")
    if dev.type not in ("cpu", "cuda"):
        raise HandoffError("--device %s: this build verifies on cpu or cuda" % device)
    # only after the cheap refusals: a refused artifact must not have touched this process's environment
    try:
        apply_kernel_env(meta.kernel_env)
    except AuditError as e:
        raise HandoffError(str(e)) from e

    from ..train.engine import TrainEngine

    cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size = V, S, R
    cfg.run.tp_size = 1  # the hash does not depend on how a tensor-parallel group split the work
    engine = TrainEngine(cfg, device, 0, 1, init=False)
    try:
        Checkpointer(checkpoint.parent.parent).load(checkpoint, engine)   # reads dcp/ through the allow-list unpickler
        result = verify_loaded_state(engine, checkpoint, expect_hash=expect_hash, prev_hash=prev_hash, include_grads=sh.include_grads,
                                     include_batch=sh.include_batch, tensor_digest=meta.tensor_digest)
    finally:
        engine.close()
    result.update(step=step, checkpoint=str(checkpoint))
    return result


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="pretrain-audit-verify-handoff",
                                description="Rebuild a hand-off checkpoint's published state hash from disk (no forward / backward pass) "
                                            "and compare it.")
    p.add_argument("--checkpoint", required=True, help="the hand-off checkpoint directory (step_<N>)")
    p.add_argument("--expect-hash", required=True, help="the PUBLISHED hash of this checkpoint's own step: a literal hex digest from the "
                                                        "run's state_hashes.jsonl, never from the artifact")
    p.add_argument("--prev-hash", required=True, help="the PUBLISHED hash of the previous HASHED step, which the chain folds in (with a "
                                                      "cadence of N: N steps back)")
    p.add_argument("--config-name", default=None, help="use this configuration instead of the one embedded in the checkpoint")
    p.add_argument("--device", default="cpu", help="where to hold the state (the digest does not depend on it)")
    p.add_argument("--json", dest="json_out", default=None, help="also write the result object to this path")
    return p


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    a = build_parser().parse_args(argv)
    from torch.distributed.checkpoint.api import CheckpointException  # a BaseException: the tensor loader wraps its failures in it

    try:
        result = verify_handoff(a.checkpoint, expect_hash=a.expect_hash, prev_hash=a.prev_hash, config_name=a.config_name, device=a.device)
    except (Exception, CheckpointException) as e:
        error = str(e) if isinstance(e, HandoffError) else "%s: %s" % (type(e).__name__, e)
        if not isinstance(e, HandoffError):
            log.exception("unexpected failure while verifying the hand-off")
        result = {"verified": False, "error": error}
    if a.json_out:
        try:
            Path(a.json_out).write_text(json.dumps(result, indent=2) + "\n")
        except OSError as e:
            result = {"verified": False, "error": "cannot write %s: %s" % (a.json_out, e)}   # fail closed: no stale file stands in
    print(json.dumps(result, indent=2), flush=True)
    if "error" in result:
        log.error("%s", result["error"])
        return 1
    if result["verified"]:
        log.info("VERIFIED tensor state: step %d reproduces the published hash %s", result["step"], result["expected_hash"])
        return 0
    from .audit_replay import mismatch_message

    print(mismatch_message(result["reconstructed_hash"], result["expected_hash"]), file=sys.stderr)
    log.error("MISMATCH: the hashed state of this hand-off is not the state the run committed to")
    return 1


if __name__ == "__main__":
    sys.exit(main())
