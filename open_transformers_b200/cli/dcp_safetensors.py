"""``pretrain-dcp-safetensors pack|unpack``: checkpoint directory <-> ONE safetensors file.

``pack`` stores every tensor of ``dcp/`` under its flattened key plus, in the header, the format tag
``pretrain.format = dcp-safetensors/1``, a *skeleton* (JSON of the non-tensor structure: optimizer steps and
param groups) and a *sidecar* (the small resume files, base64: meta.json, state_hash.txt, global_stream.json,
spike_protocol.json, batch_hasher.rank_*.bin, rng.rank_*.pt). ``unpack`` rebuilds a directory a run can resume
from or an auditor can replay. Only allow-listed sidecar names are ever written
(reference src/pretrain/cli/dcp_safetensors.py:80-252)."""
from __future__ import annotations

import argparse
import base64
import json
import re
import sys
from pathlib import Path

FORMAT = "dcp-safetensors/1"
SIDECAR_ALLOW = re.compile(r"^(meta\.json|state_hash\.txt|global_stream\.json|spike_protocol\.json|batch_hasher\.rank_\d+\.bin|rng\.rank_\d+\.pt)$")


def pack(ckpt_dir: str, out_file: str) -> dict:
    import torch
    import torch.distributed.checkpoint as dcp
    from safetensors.torch import save_file
    from torch.distributed.checkpoint.metadata import BytesStorageMetadata, TensorStorageMetadata

    from ..train.checkpoint import COMPLETE, validate_dcp_metadata

    d = Path(ckpt_dir)
    if not (d / COMPLETE).exists():
        raise FileNotFoundError("%s is not a complete checkpoint" % d)
    validate_dcp_metadata(d / "dcp")
    reader = dcp.FileSystemReader(str(d / "dcp"))
    md = reader.read_metadata()
    tensors = {k: torch.empty(m.size, dtype=m.properties.dtype) for k, m in md.state_dict_metadata.items()
               if isinstance(m, TensorStorageMetadata)}
    dcp.load(tensors, storage_reader=reader, no_dist=True)
    meta = json.loads((d / "meta.json").read_text())
    skeleton = {"tensor_keys": sorted(tensors), "bytes_keys": sorted(k for k, m in md.state_dict_metadata.items() if isinstance(m, BytesStorageMetadata))}
    steps = {k: int(v) for k, v in tensors.items() if k.endswith(".step")}
    skeleton["optimizer_steps"] = steps
    sidecar = {p.name: base64.b64encode(p.read_bytes()).decode() for p in sorted(d.iterdir()) if p.is_file() and SIDECAR_ALLOW.match(p.name)}
    header = {"pretrain.format": FORMAT, "pretrain.skeleton": json.dumps(skeleton, sort_keys=True), "pretrain.sidecar": json.dumps(sidecar, sort_keys=True),
              "pretrain.step": str(meta.get("step", 0))}
    Path(out_file).parent.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, out_file, metadata=header)
    return {"file": out_file, "tensors": len(tensors), "sidecar_files": sorted(sidecar)}


def unpack(in_file: str, out_dir: str) -> dict:
    import torch
    import torch.distributed.checkpoint as dcp
    from safetensors import safe_open

    from ..train.checkpoint import COMPLETE

    with safe_open(in_file, framework="pt") as f:
        md = f.metadata() or {}
        if md.get("pretrain.format") != FORMAT:
            raise ValueError("%s: not a %s file (pretrain.format=%r)" % (in_file, FORMAT, md.get("pretrain.format")))
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    sidecar = json.loads(md.get("pretrain.sidecar", "{}"))
    for name in sidecar:  # names come from an untrusted header: checked before anything is written
        if not isinstance(name, str) or not SIDECAR_ALLOW.match(name):
            raise ValueError("sidecar entry %r is not an allowed file name" % (name,))
    d = Path(out_dir)
    (d / "dcp").mkdir(parents=True, exist_ok=True)
    nested: dict = {}
    for k, v in tensors.items():
        # keys were flattened by DCP with "." separators at the TOP levels only: model.<name>, optim.state.<name>.<field>
        if k.startswith("model."):
            nested.setdefault("model", {})[k[len("model."):]] = v
        elif k.startswith("optim.state."):
            name, field = k[len("optim.state."):].rsplit(".", 1)
            nested.setdefault("optim", {}).setdefault("state", {}).setdefault(name, {})[field] = v
        else:
            nested[k] = v
    meta = json.loads(base64.b64decode(sidecar["meta.json"])) if "meta.json" in sidecar else {}
    if "optim" in nested:
        pg_src = meta.get("param_groups")
        nested["optim"]["param_groups"] = pg_src if pg_src else []
    dcp.save(nested, storage_writer=dcp.FileSystemWriter(str(d / "dcp"), thread_count=1), no_dist=True)
    written = []
    for name, b64 in sidecar.items():
        (d / name).write_bytes(base64.b64decode(b64))
        written.append(name)
    (d / COMPLETE).write_text("unpacked\n")
    return {"dir": str(d), "tensors": len(tensors), "sidecar_files": sorted(written)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-dcp-safetensors")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pack"); p.add_argument("checkpoint"); p.add_argument("out")
    u = sub.add_parser("unpack"); u.add_argument("file"); u.add_argument("out_dir")
    a = ap.parse_args(argv)
    res = pack(a.checkpoint, a.out) if a.cmd == "pack" else unpack(a.file, a.out_dir)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
