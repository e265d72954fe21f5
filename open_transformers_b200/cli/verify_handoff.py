"""``pretrain-audit-verify-handoff``: does a downloaded hand-off hold the state the run committed to? Answered from the
files alone, in seconds plus one checkpoint load, with no forward or backward pass and no training data.

What a hand-off is: a checkpoint directory plus ``gradients.safetensors``. The chained state hash covers weights, AdamW
moments, parameter groups, the step's post-clip gradients and the running batch digest; an ordinary checkpoint has all of
these except the gradients, which is why the replay writes them beside a checkpoint it hands on.

What the verifier does, cheapest question first (``Handoff.plan``): are the two commitments real digests; is the directory
complete; is its step one the run hashed; does what the directory says about itself agree with the commitments; is the
recorded topology sane; are the files the hash needs all there. Only then the recorded kernel switches are applied, the
engine is built in the recorded virtual topology, ``dcp/`` is loaded through the allow-list reader, the gradients are put
back bit for bit and the hash is recomputed (``verify_loaded_state``).

Trust: ``--expect-hash`` (the checkpoint's own step) and ``--prev-hash`` (the previous hashed step) are typed in by the
caller from the run's published ``logs/state_hashes.jsonl``. Nothing inside the directory can stand in for them -
``state_hash.txt`` is written by the same hand that wrote the tensors - so file paths are not accepted for either, and
``state_hash.txt`` is consulted only to stop early when it already contradicts the published value. The switches read from
``meta.json`` (cadence, gradient / batch inclusion, shard count) need no trust either: each of them changes the digest, so a
false one fails the comparison. Outside the hash, hence outside a match: RNG state, the stream cursor, spike state.

(reference src/pretrain/cli/verify_handoff.py; gradient file format src/pretrain/cli/audit_replay.py:765-798)"""
from __future__ import annotations

import argparse
import dataclasses
import json
import logging
import re
import sys
from pathlib import Path

GRAD_FILE = "gradients.safetensors"
GRAD_FORMAT = "pretrain-audit-gradients"
GRAD_VERSION = "1"
_HEX64 = re.compile(r"[0-9a-fA-F]{64}")
log = logging.getLogger("pretrain.audit.verify")


class HandoffError(Exception):
    """A reason not to spend a replay on this directory."""


# ------------------------------------------------------------------------------------------- gradient file
def write_gradient_sidecar(ckpt_dir, named_grads: dict) -> Path:
    """One tensor per parameter with a gradient; parameters without one are NAMED in the header (``none_grad_names``), so
    that "no entry" never means "no gradient"."""
    from safetensors.torch import save_file

    have = {n: g.detach().to("cpu").contiguous().clone() for n, g in named_grads.items() if g is not None}
    without = sorted(n for n, g in named_grads.items() if g is None)
    path = Path(ckpt_dir) / GRAD_FILE
    save_file(have, str(path), metadata={"format": GRAD_FORMAT, "format_version": GRAD_VERSION, "none_grad_names": json.dumps(without)})
    return path


def read_gradient_sidecar(ckpt_dir) -> dict:
    """``{parameter name: fp32 tensor, or None for a named absence}``. Whatever is wrong with the file - not there, not
    safetensors, another format tag, a header that does not parse, a name listed twice or on both sides - is a
    ``HandoffError`` that says so."""
    import safetensors

    path = Path(ckpt_dir) / GRAD_FILE
    if not path.is_file():
        raise HandoffError("%s is missing. The hash includes the step's gradients; without the file it cannot be recomputed, and a "
                           "missing file is not the same as a model whose gradients were all None. This is not a hand-off." % path)
    try:
        with safetensors.safe_open(str(path), framework="pt", device="cpu") as f:
            header = f.metadata() or {}
            tag = (header.get("format"), header.get("format_version"))
            if tag != (GRAD_FORMAT, GRAD_VERSION):
                raise HandoffError("%s: format tag %r, this verifier reads %r" % (path, tag, (GRAD_FORMAT, GRAD_VERSION)))
            absent = json.loads(header["none_grad_names"])
            if not (isinstance(absent, list) and all(isinstance(n, str) for n in absent)):
                raise HandoffError("%s: none_grad_names is not a list of names" % path)
            out: dict = {name: f.get_tensor(name) for name in f.keys()}
    except (OSError, ValueError, KeyError, safetensors.SafetensorError) as e:
        raise HandoffError("%s does not parse as a gradient file (%s: %s)" % (path, type(e).__name__, e)) from e
    if len(absent) != len(set(absent)):
        raise HandoffError("%s: a name appears twice in none_grad_names" % path)
    clash = sorted(set(absent) & set(out))
    if clash:
        raise HandoffError("%s: %s has a tensor AND is listed as having no gradient" % (path, ", ".join(clash[:4])))
    out.update(dict.fromkeys(absent))
    return out


def attach_gradients(engine, grads: dict, where: str = GRAD_FILE) -> int:
    """Put a hand-off's gradients into the engine's reduced-gradient buffer, bytes untouched; returns how many tensors went
    in. The file must speak for every parameter of THIS model exactly once, in fp32 and in the parameter's shape - a file
    made for another model is turned away here, with the name, rather than surfacing as a bare mismatch later."""
    import torch

    lay = engine.layout
    want = {n: tuple(lay.shapes[i]) for i, n in enumerate(engine.names)}
    unknown, unspoken = sorted(set(grads) - set(want)), sorted(set(want) - set(grads))
    if unknown:
        raise HandoffError("%s names parameters the model does not have: %s" % (where, ", ".join(unknown[:4])))
    if unspoken:
        raise HandoffError("%s says nothing about %s (no tensor, no none_grad_names entry): incomplete" % (where, ", ".join(unspoken[:4])))
    for n, g in grads.items():
        if g is not None and (g.dtype, tuple(g.shape)) != (torch.float32, want[n]):
            raise HandoffError("%s: %s comes as %s %s; the model's gradient is torch.float32 %s" % (where, n, g.dtype, tuple(g.shape), want[n]))
    engine.grad_red.zero_()
    count = 0
    for i, n in enumerate(engine.names):
        if grads[n] is not None:
            lay.view(engine.grad_red, i).copy_(grads[n])
            count += 1
    return count


# ------------------------------------------------------------------------------------------- batch chains
def read_batch_digest(ckpt_dir, dp_world_size: int) -> bytes:
    """The run's batch digest: the 32-byte chains of virtual ranks 0 .. dp_world_size-1, combined in that order (one rank:
    its chain as it is). All of them or nothing - hashing fewer would be another formula, and its mismatch a false alarm."""
    from ..train.state_hash import combine_batch_digests

    chains = []
    for v in range(dp_world_size):
        f = Path(ckpt_dir) / ("batch_hasher.rank_%d.bin" % v)
        if not f.is_file():
            raise HandoffError("%s is missing; with dp_world_size=%d the hash needs the batch chain of each of the %d ranks"
                               % (f, dp_world_size, dp_world_size))
        chain = f.read_bytes()
        if len(chain) != 32:
            raise HandoffError("%s holds %d bytes, a chain is 32" % (f, len(chain)))
        chains.append(chain)
    return combine_batch_digests(chains)


# ------------------------------------------------------------------------------------------- the cheap questions
@dataclasses.dataclass
class Plan:
    """What the expensive part needs, established without loading a tensor."""
    cfg: object
    step: int
    world: int
    replicate: int
    shard: int
    expect_hash: str
    prev_hash: str
    tensor_digest: str
    kernel_env: dict


class Handoff:
    def __init__(self, path):
        self.path = Path(path)

    def literal(self, flag: str, value) -> str:
        if not isinstance(value, str) or not _HEX64.fullmatch(value.strip()):
            raise HandoffError("%s takes the 64 hex digits of a published hash, typed out: no file path, no shortened form" % flag)
        return value.strip().lower()

    def meta(self) -> dict:
        f = self.path / "meta.json"
        if not f.is_file():
            raise HandoffError("%s is missing, so neither topology nor hash cadence of this directory is known" % f)
        if not (self.path / "_COMPLETE").is_file():
            raise HandoffError("%s has no _COMPLETE marker: an unfinished save or a partial download" % self.path)
        try:
            meta = json.loads(f.read_text())
        except (OSError, ValueError) as e:
            raise HandoffError("%s is not readable JSON (%s)" % (f, e)) from e
        if not isinstance(meta, dict):
            raise HandoffError("%s: expected a JSON object" % f)
        if type(meta.get("step")) is not int or meta["step"] < 1:
            raise HandoffError("%s: step has to be a positive integer, found %r" % (f, meta.get("step")))
        return meta

    def plan(self, expect_hash, prev_hash, config_name: str | None = None) -> Plan:
        from ..config import load_config, parse_config_resolved
        from ..train.checkpoint import CheckpointMeta
        from .audit_replay import MAX_AUDIT_WORLD

        expect = self.literal("--expect-hash", expect_hash)
        prev = self.literal("--prev-hash", prev_hash)
        raw = self.meta()
        known = CheckpointMeta.from_json(json.dumps(raw))
        cfg = load_config(config_name) if config_name else parse_config_resolved(known.config_resolved)
        every, step = cfg.train.state_hash.every_n_steps, raw["step"]
        if every < 1:
            raise HandoffError("this run never hashed its state (state_hash.every_n_steps = %d): nothing was published to compare with" % every)
        if step % every:
            raise HandoffError("step %d lies between hashed steps (cadence %d). The published log has no entry for it, and its "
                               "state_hash.txt is a side link that the chain does not pass through: unsupported" % (step, every))
        note = self.path / "state_hash.txt"
        if note.is_file():
            said, chain = note.read_text().strip().lower(), str(raw.get("chained_hash") or "").lower()
            if said != chain:
                raise HandoffError("%s (%s...) is not the running chain recorded in meta.json (%s...): on a hashed step the two are one "
                                   "value, so this is a side link or an edited file" % (note, said[:16], chain[:16]))
            if said != expect:
                raise HandoffError("the directory and the published log disagree about step %d before any tensor is read:\n"
                                   "    state_hash.txt  %s\n    published       %s\nthe log wins; not worth a replay" % (step, said, expect))
        world = raw.get("dp_world_size") or 1
        replicate, shard = raw.get("dp_replicate") or 1, raw.get("dp_shard") or world
        sizes = (world, replicate, shard)
        if not all(type(x) is int for x in sizes) or min(sizes) < 1 or world > MAX_AUDIT_WORLD:
            raise HandoffError("recorded topology dp_world_size=%r dp_replicate=%r dp_shard=%r is implausible (integers from 1, world at most %d)"
                               % (world, replicate, shard, MAX_AUDIT_WORLD))
        if replicate * shard != world:
            raise HandoffError("recorded topology does not multiply out: %d replicas x %d shards is not %d ranks" % (replicate, shard, world))
        if cfg.train.state_hash.include_batch:
            read_batch_digest(self.path, world)
        if cfg.train.state_hash.include_grads and not (self.path / GRAD_FILE).is_file():
            read_gradient_sidecar(self.path)   # raises with the full explanation
        return Plan(cfg, step, world, replicate, shard, expect, prev, known.tensor_digest, known.kernel_env)


# ------------------------------------------------------------------------------------------- the comparison
def verify_loaded_state(engine, checkpoint, *, expect_hash: str, prev_hash: str, include_grads: bool, include_batch: bool,
                        tensor_digest: str = "raw") -> dict:
    """Recompute and compare, given an engine that already holds the checkpoint's weights and moments. Whatever happens,
    the gradient buffer is zero again afterwards: they are as large as the model and belong to the finished step."""
    checkpoint = Path(checkpoint)
    attached = None
    try:
        if include_grads:
            attached = attach_gradients(engine, read_gradient_sidecar(checkpoint), str(checkpoint / GRAD_FILE))
        batch = read_batch_digest(checkpoint, engine.V) if include_batch else None
        rebuilt = engine.sharded_state_hash(prev_hash, batch, include_grads=include_grads, tensor_digest=tensor_digest)
    finally:
        engine.grad_red.zero_()
    return {"verified": rebuilt == expect_hash, "reconstructed_hash": rebuilt, "expected_hash": expect_hash, "prev_hash": prev_hash,
            "dp_world_size": engine.V, "dp_shard": engine.dp_shard, "include_grads": include_grads, "include_batch": include_batch,
            "gradients_attached": attached}


def verify_handoff(checkpoint, *, expect_hash: str, prev_hash: str, config_name: str | None = None, device: str = "cpu") -> dict:
    """The whole check; the result's ``verified`` says whether the directory reproduces ``expect_hash``. Raises
    ``HandoffError`` where the question cannot even be put."""
    import torch

    from ..train.checkpoint import Checkpointer
    from .audit_replay import AuditError, apply_kernel_env

    ho = Handoff(checkpoint)
    plan = ho.plan(expect_hash, prev_hash, config_name)
    kind = torch.device(device).type
    if kind not in ("cpu", "cuda"):
        raise HandoffError("--device %s: the state can be held on cpu or cuda" % device)
    if kind == "cuda" and not torch.cuda.is_available():
        raise HandoffError("--device %s: no CUDA device here; cpu gives the same digest" % device)
    try:
        apply_kernel_env(plan.kernel_env)   # last of the preliminaries: a directory that was turned away has changed nothing here
    except AuditError as e:
        raise HandoffError(str(e)) from e

    from ..train.engine import TrainEngine

    run = plan.cfg.run
    run.virtual_dp_size, run.dp_shard_size, run.dp_replicate_size, run.tp_size = plan.world, plan.shard, plan.replicate, 1
    sh = plan.cfg.train.state_hash
    engine = TrainEngine(plan.cfg, device, 0, 1, init=False)
    try:
        Checkpointer(ho.path.parent.parent).load(ho.path, engine)
        out = verify_loaded_state(engine, ho.path, expect_hash=plan.expect_hash, prev_hash=plan.prev_hash, include_grads=sh.include_grads,
                                  include_batch=sh.include_batch, tensor_digest=plan.tensor_digest)
    finally:
        engine.close()
    out.update(step=plan.step, checkpoint=str(ho.path))
    return out


# ------------------------------------------------------------------------------------------- command line
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="pretrain-audit-verify-handoff", description=__doc__.split("\n\n")[0])
    p.add_argument("--checkpoint", required=True, help="hand-off directory (…/step_<N>)")
    p.add_argument("--expect-hash", required=True, help="published hash of that step, 64 hex digits copied from state_hashes.jsonl")
    p.add_argument("--prev-hash", required=True, help="published hash of the hashed step before it (cadence N: N steps earlier)")
    p.add_argument("--config-name", default=None, help="a named configuration instead of the embedded one")
    p.add_argument("--device", default="cpu", help="cpu (default) or cuda; the digest is the same")
    p.add_argument("--json", dest="json_out", default=None, metavar="FILE", help="write the result object here as well")
    return p


def main(argv=None) -> int:
    """Exit status 0 only for a verified hand-off. The result object always goes to standard output (and ``--json``); a
    refusal or crash is ``{"verified": false, "error": ...}``, so a stale file from an earlier run never answers for this one."""
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s :: %(message)s")
    a = build_parser().parse_args(argv)
    from torch.distributed.checkpoint.api import CheckpointException   # not an Exception subclass; the tensor reader raises it

    try:
        result = verify_handoff(a.checkpoint, expect_hash=a.expect_hash, prev_hash=a.prev_hash, config_name=a.config_name, device=a.device)
    except HandoffError as e:
        result = {"verified": False, "error": str(e)}
    except (Exception, CheckpointException) as e:
        log.exception("verification stopped on an error that is not a refusal")
        result = {"verified": False, "error": "%s: %s" % (type(e).__name__, e)}
    if a.json_out:
        try:
            Path(a.json_out).write_text(json.dumps(result, indent=2) + "\n")
        except OSError as e:
            result = {"verified": False, "error": "cannot write %s: %s" % (a.json_out, e)}
    print(json.dumps(result, indent=2), flush=True)
    if "error" in result:
        log.error("%s", result["error"])
    elif result["verified"]:
        log.info("VERIFIED: step %d reproduces %s", result["step"], result["expected_hash"])
        return 0
    else:
        from .audit_replay import mismatch_message

        print(mismatch_message(result["reconstructed_hash"], result["expected_hash"]), file=sys.stderr)
    return 1


if __name__ == "__main__":
    sys.exit(main())
