"""``python -m open_transformers_b200.cli.hash_ckpt DIR``: v2 full-tensor fingerprint of a checkpoint
(weights + optimizer step and moments + param groups), independent of any topology
(reference src/pretrain/cli/hash_ckpt.py:56-134)."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def hash_checkpoint(ckpt_dir: str, include_optimizer: bool = True) -> str:
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
    ap.add_argument("--weights-only", action="store_true")
    a = ap.parse_args(argv)
    print(hash_checkpoint(a.checkpoint, include_optimizer=not a.weights_only))
    return 0


if __name__ == "__main__":
    sys.exit(main())
