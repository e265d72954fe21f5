"""``pretrain-audit-verify-handoff``: recompute a checkpoint's state hash from disk alone (no forward or
backward): weights + moments from ``dcp/``, post-clip gradients from ``gradients.safetensors``, the batch term
from the per-rank ``batch_hasher.rank_<v>.bin`` files, the previous link from ``--prev-hash``. A relay of
auditors can thus accept a hand-off checkpoint before spending compute on it
(reference src/pretrain/cli/verify_handoff.py:73-391)."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

GRAD_FORMAT = "pretrain-audit-gradients"


def write_gradient_sidecar(ckpt_dir, named_grads: dict) -> Path:
    from safetensors.torch import save_file

    tensors, none_names = {}, []
    for name, g in named_grads.items():
        if g is None:
            none_names.append(name)
        else:
            tensors[name] = g.detach().to("cpu").contiguous().clone()
    p = Path(ckpt_dir) / "gradients.safetensors"
    save_file(tensors, str(p), metadata={"format": GRAD_FORMAT, "format_version": "1", "none_grad_names": json.dumps(sorted(none_names))})
    return p


def read_gradient_sidecar(ckpt_dir) -> dict:
    from safetensors import safe_open

    p = Path(ckpt_dir) / "gradients.safetensors"
    if not p.is_file():
        raise FileNotFoundError("%s missing: this checkpoint is not an audit hand-off" % p)
    out = {}
    with safe_open(str(p), framework="pt") as f:
        md = f.metadata() or {}
        if md.get("format") != GRAD_FORMAT or md.get("format_version") != "1":
            raise ValueError("%s: unexpected format %r / version %r" % (p, md.get("format"), md.get("format_version")))
        for k in f.keys():
            out[k] = f.get_tensor(k)
        for k in json.loads(md.get("none_grad_names", "[]")):
            out[k] = None
    return out


def read_batch_digest(ckpt_dir, dp_world_size: int) -> bytes:
    from ..train.state_hash import combine_batch_digests

    chains = []
    for v in range(dp_world_size):
        p = Path(ckpt_dir) / ("batch_hasher.rank_%d.bin" % v)
        if not p.is_file():
            raise FileNotFoundError("%s missing" % p)
        b = p.read_bytes()
        if len(b) != 32:
            raise ValueError("%s holds %d bytes, expected 32" % (p, len(b)))
        chains.append(b)
    return combine_batch_digests(chains)


def verify_handoff(checkpoint: str, expect_hash: str | None = None, prev_hash: str | None = None, config_name: str | None = None,
                   device: str = "cpu") -> dict:
    from ..config import load_config, parse_config_resolved
    from ..train.checkpoint import Checkpointer
    from ..train.engine import TrainEngine

    meta = Checkpointer.read_meta(checkpoint)
    cfg = load_config(config_name) if config_name else parse_config_resolved(meta.config_resolved)
    cfg.run.virtual_dp_size, cfg.run.dp_shard_size, cfg.run.dp_replicate_size = meta.dp_world_size, meta.dp_shard, meta.dp_replicate
    cfg.run.tp_size = 1  # the hash does not depend on how a tensor-parallel group split the work
    engine = TrainEngine(cfg, device, 0, 1, init=False)
    Checkpointer(Path(checkpoint).parent.parent).load(checkpoint, engine)
    grads = read_gradient_sidecar(checkpoint)
    lay = engine.layout
    for i, n in enumerate(engine.names):
        if n not in grads:
            raise KeyError("gradient sidecar lacks %s" % n)
        if grads[n] is not None:
            lay.view(engine.grad_red, i).copy_(grads[n])
    bd = read_batch_digest(checkpoint, meta.dp_world_size) if cfg.train.state_hash.include_batch else None
    got = engine.sharded_state_hash(prev_hash, bd, include_grads=cfg.train.state_hash.include_grads, tensor_digest=meta.tensor_digest)
    want = expect_hash
    if want is None and (Path(checkpoint) / "state_hash.txt").is_file():
        want = (Path(checkpoint) / "state_hash.txt").read_text().strip()
    engine.close()
    return {"checkpoint": str(checkpoint), "step": meta.step, "state_hash": got, "expected": want, "match": (got == want) if want else None}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-audit-verify-handoff")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--expect-hash")
    ap.add_argument("--prev-hash")
    ap.add_argument("--config-name")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    from .audit_replay import mismatch_message, resolve_expect_hash

    res = verify_handoff(a.checkpoint, resolve_expect_hash(a.expect_hash), resolve_expect_hash(a.prev_hash), a.config_name, a.device)
    print(json.dumps(res, indent=1) if a.json else "MATCH=%s state_hash=%s" % (res["match"], res["state_hash"]))
    if res["match"] is False:
        print(mismatch_message(res["state_hash"], res["expected"]), file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
