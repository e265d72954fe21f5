"""``python -m open_transformers_b200.cli.hash_ckpt DIR``: v2 full-tensor fingerprint of a checkpoint
(weights + optimizer step and moments + param groups), independent of any topology
(reference src/pretrain/cli/hash_ckpt.py:56-134)."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def check_against_config(params: dict, config_name: str, overrides: list[str]) -> None:
    """The checkpoint's parameter names and shapes against the model a named configuration describes (built without
    storage). The fingerprint itself needs no configuration - it reads the tensors as stored - so this is what
    ``--config-name`` adds: hashing a checkpoint under the wrong recipe fails instead of printing a digest."""
    import torch

    from ..config import load_config
    from ..models.llama3 import build_model

    cfg = load_config(config_name, list(overrides or []))
    with torch.device("meta"):
        model = build_model(cfg.model)
    want = {n: tuple(p.shape) for n, p in model.named_parameters()}
    have = {n: tuple(t.shape) for n, t in params.items()}
    if want != have:
        missing, extra = sorted(set(want) - set(have)), sorted(set(have) - set(want))
        differ = sorted(n for n in set(want) & set(have) if want[n] != have[n])
        raise ValueError("checkpoint does not match configuration %s: %d parameters missing (%s), %d not in the model (%s), %d with "
                         "another shape (%s)" % (config_name, len(missing), ", ".join(missing[:3]), len(extra), ", ".join(extra[:3]),
                                                 len(differ), ", ".join(differ[:3])))


def hash_checkpoint(ckpt_dir: str, include_optimizer: bool = True, config_name: str | None = None, overrides: list[str] | None = None) -> str:
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata
    import torch

    from ..train import state_hash as SH
    from ..train.checkpoint import optimizer_state_names, validate_dcp_metadata

    d = Path(ckpt_dir) / "dcp"
    validate_dcp_metadata(d)
    reader = dcp.FileSystemReader(str(d))
    md = reader.read_metadata()
    template = {}
    for key, m in md.state_dict_metadata.items():
        if isinstance(m, TensorStorageMetadata):
            # keys are flattened "model.<name>" / "optim.state.<name>.<field>": keep them flat
            template[key] = torch.empty(m.size, dtype=m.properties.dtype)
    dcp.load(template, storage_reader=reader, no_dist=True)
    params = {k[len("model."):]: v for k, v in template.items() if k.startswith("model.")}
    if config_name is not None:
        check_against_config(params, config_name, overrides or [])
    opt = {}
    if include_optimizer:
        by_index = optimizer_state_names(ckpt_dir)  # torch-style payload: optim.state.<index>; older ones are keyed by name
        for k, v in template.items():
            if k.startswith("optim.state."):
                name, field = k[len("optim.state."):].rsplit(".", 1)
                opt.setdefault(by_index.get(name, name), {})[field] = v
    return SH.compute_state_hash(list(params.items()), opt or None, None)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hash_ckpt")
    ap.add_argument("checkpoint")
    ap.add_argument("--weights-only", action="store_true", help="leave the optimizer state out (comparisons across optimizer changes)")
    ap.add_argument("--config-name", default=None, help="check the checkpoint against this configuration's model before hashing")
    ap.add_argument("--override", nargs="*", default=[], help="key=value overrides of --config-name")
    a = ap.parse_args(argv)
    print(hash_checkpoint(a.checkpoint, include_optimizer=not a.weights_only, config_name=a.config_name, overrides=a.override))
    return 0


if __name__ == "__main__":
    sys.exit(main())
