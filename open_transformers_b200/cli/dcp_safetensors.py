"""``pretrain-dcp-safetensors``: a DCP checkpoint <-> ONE safetensors file, both ways, offline.

    pretrain-dcp-safetensors to-safetensors   CKPT_DIR out.safetensors [--keys model ...] [--verify]
    pretrain-dcp-safetensors from-safetensors in.safetensors OUT_DIR   [--top-level-key model] [--verify]

``CKPT_DIR`` is a ``step_N`` directory (with ``dcp/`` inside) or a bare DCP directory. Every tensor leaf of the state
dict becomes one safetensors entry under its dotted name (``model.blocks.0.attn.wq.weight``, ``optim.state.3.exp_avg``);
the nesting and every non-tensor leaf (``param_groups``, counters) travel as a JSON *skeleton* in the header
(``pretrain.skeleton``), so the way back is lossless and no dtype is touched. For a ``step_N`` directory the small
resume files travel too, as a *sidecar* (``pretrain.sidecar``): ``meta.json``, ``state_hash.txt``, ``global_stream.json``,
``spike_protocol.json``, ``sampler.rank_N.json``, ``batch_hasher.rank_N.bin``, the per-rank RNG states (decoded to tensors:
no pickle is embedded) and a hand-off's ``gradients.safetensors``. ``from-safetensors`` then rebuilds a complete checkpoint
directory (``dcp/`` written as one full-tensor shard, which DCP re-shards on load, + the sidecar files + ``_COMPLETE``)
that ``--resume-from`` and ``pretrain-audit-replay --checkpoint`` accept. With ``--keys`` or a bare DCP directory only
tensors travel and the way back gives a bare DCP directory. A foreign file without a skeleton becomes a flat state dict,
nested under ``--top-level-key`` if given.

Checkpoints and safetensors headers are untrusted input: the DCP ``.metadata`` pickle passes the allow-list gate of
``train/checkpoint.py`` before anything is read, non-tensor leaves are unpickled with ``weights_only=True``, sidecar
names from a header must match an exact allow-list before they become paths, and a non-empty output directory is refused.
``--verify`` re-reads what was written and compares it with what was meant to be written, bit for bit (NaN == NaN).

Header format and CLI surface: reference src/pretrain/cli/dcp_safetensors.py:80-92, 170-252, 630-700.
``pack`` / ``unpack`` are the same two operations as functions.
"""
from __future__ import annotations

import argparse
import base64
import io
import json
import math
import re
import sys
from pathlib import Path
from typing import Any

FORMAT_KEY, FORMAT = "pretrain.format", "dcp-safetensors/1"
SKELETON_KEY, SIDECAR_KEY = "pretrain.skeleton", "pretrain.sidecar"
SIDECAR_FILE = re.compile(r"^(meta\.json|global_stream\.json|spike_protocol\.json|state_hash\.txt|sampler\.rank_\d+\.json"
                          r"|batch_hasher\.rank_\d+\.bin)$")
GRADIENTS = "gradients.safetensors"


class ConversionError(ValueError):
    """Anything the user has to fix (wrong directory, refused header, failed verification); the command prints it and exits 2."""


# ------------------------------------------------------------------------------------------- offline DCP access
def resolve_dcp_dir(path: Path) -> Path:
    for cand in (path / "dcp", path):
        if (cand / ".metadata").is_file():
            return cand
    raise ConversionError("%s is not a DCP checkpoint (no dcp/.metadata and no .metadata in it)" % path)


def read_dcp(dcp_dir: Path) -> dict:
    """The full nested state dict of a DCP directory, rebuilt from its metadata alone (no model, no process group)."""
    import torch
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    from ..train.checkpoint import validate_dcp_metadata

    validate_dcp_metadata(dcp_dir)
    reader = dcp.FileSystemReader(str(dcp_dir))
    md = reader.read_metadata()

    class SafeBytesPlanner(dcp.DefaultLoadPlanner):
        def load_bytes(self, read_item, value: io.BytesIO) -> None:  # the stock planner unpickles these without a gate
            self.state_dict[read_item.dest_index.fqn] = torch.load(value, weights_only=True)

    flat = {k: (torch.empty(m.size, dtype=m.properties.dtype) if isinstance(m, TensorStorageMetadata) else None)
            for k, m in md.state_dict_metadata.items()}
    planner = SafeBytesPlanner(flatten_state_dict=False)
    dcp.load(flat, storage_reader=reader, planner=planner, no_dist=True)
    flat = dict(planner.state_dict)  # the non-tensor leaves land in the planner's copy
    # DCP records, per flattened name, the path it came from: a string is a dictionary key (it turns every mapping key
    # into a string, `optim.state.3` included), an integer is a list index
    paths = md.planner_data or {}
    root: dict = {}
    for key, value in flat.items():
        path = tuple(paths.get(key, (key,)))
        node: Any = root
        for part, nxt in zip(path[:-1], path[1:]):
            fresh: Any = [] if isinstance(nxt, int) else {}
            if isinstance(part, int):
                while len(node) <= part:
                    node.append(None)
                if node[part] is None:
                    node[part] = fresh
                node = node[part]
            else:
                node = node.setdefault(part, fresh)
        last = path[-1]
        if isinstance(last, int):
            while len(node) <= last:
                node.append(None)
            node[last] = value
        else:
            node[last] = value
    return root


def write_dcp(state: dict, dcp_dir: Path) -> None:
    import torch.distributed.checkpoint as dcp

    dcp.save(state, storage_writer=dcp.FileSystemWriter(str(dcp_dir), thread_count=1), no_dist=True)


# ------------------------------------------------------------------------------------- state dict <-> skeleton + tensors
class _Encoder:
    """Walks a state dict once: tensors go to `self.tensors` under their dotted path, the structure and the plain values
    become the skeleton. Node forms: {"t": "tensor", "key"}, {"t": "dict", "items": [[key, node], ...]}, {"t": "list" |
    "tuple", "items": [...]}, {"t": "v", "v": scalar}, {"t": "float", "v": repr} for inf / nan, {"t": "bytes", "v": base64}."""

    def __init__(self, tensors: dict | None = None):
        self.tensors = {} if tensors is None else tensors

    def _tensor_key(self, path: tuple) -> str:
        stem = ".".join(str(p) for p in path) or "_root"
        key, n = stem, 1
        while key in self.tensors:
            n += 1
            key = "%s#%d" % (stem, n)
        return key

    def encode(self, obj: Any, path: tuple = ()) -> dict:
        import torch

        where = ".".join(map(str, path)) or "<root>"
        if isinstance(obj, torch.Tensor):
            key = self._tensor_key(path)
            self.tensors[key] = obj.detach().to("cpu").contiguous()
            return {"t": "tensor", "key": key}
        if isinstance(obj, dict):
            for k in obj:
                if not (k is None or isinstance(k, (str, int, bool))):
                    raise TypeError("dictionary key %r at %s cannot be written to a skeleton" % (k, where))
            return {"t": "dict", "items": [[k, self.encode(v, path + (k,))] for k, v in obj.items()]}
        if isinstance(obj, (list, tuple)):
            return {"t": "tuple" if isinstance(obj, tuple) else "list", "items": [self.encode(v, path + (i,)) for i, v in enumerate(obj)]}
        if isinstance(obj, bytes):
            return {"t": "bytes", "v": base64.b64encode(obj).decode("ascii")}
        if isinstance(obj, float) and not math.isfinite(obj):
            return {"t": "float", "v": repr(obj)}
        if obj is None or isinstance(obj, (bool, int, float, str)):
            return {"t": "v", "v": obj}
        raise TypeError("a %s at %s cannot be written to a skeleton" % (type(obj).__name__, where))


def decode(node: dict, tensors: dict) -> Any:
    kind = node["t"]
    if kind == "tensor":
        if node["key"] not in tensors:
            raise KeyError("the skeleton names tensor %r, which the file does not hold (truncated or edited?)" % node["key"])
        return tensors[node["key"]]
    if kind == "dict":
        return {k: decode(v, tensors) for k, v in node["items"]}
    if kind in ("list", "tuple"):
        seq = [decode(v, tensors) for v in node["items"]]
        return tuple(seq) if kind == "tuple" else seq
    if kind == "v":
        return node["v"]
    if kind == "float":
        return float(node["v"])
    if kind == "bytes":
        return base64.b64decode(node["v"])
    raise ValueError("unknown skeleton node %r" % kind)


def tensor_keys(node: dict) -> set:
    if node["t"] == "tensor":
        return {node["key"]}
    if node["t"] == "dict":
        return set().union(*[tensor_keys(v) for _, v in node["items"]]) if node["items"] else set()
    if node["t"] in ("list", "tuple"):
        return set().union(*[tensor_keys(v) for v in node["items"]]) if node["items"] else set()
    return set()


def same_bits(a, b) -> bool:
    """Tensors equal as bytes (so NaN equals NaN and -0.0 differs from 0.0), same dtype and shape."""
    import torch

    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    if a.numel() == 0:
        return True
    return torch.equal(a.detach().cpu().contiguous().reshape(-1).view(torch.uint8), b.detach().cpu().contiguous().reshape(-1).view(torch.uint8))


def same_state(a: Any, b: Any) -> bool:
    import torch

    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and same_bits(a, b)
    if isinstance(a, dict) and isinstance(b, dict):
        return a.keys() == b.keys() and all(same_state(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        return len(a) == len(b) and all(same_state(x, y) for x, y in zip(a, b))
    return type(a) is type(b) and a == b


# ---------------------------------------------------------------------------------------------------------- sidecar
def collect_sidecar(ckpt_dir: Path) -> dict | None:
    """{"files": {name: text | bytes}, "rng": {rank: {"cpu", "cuda"}}, "grads": {"tensors", "metadata"} | None} of a
    ``step_N`` directory; None when it holds none of these (a bare DCP directory)."""
    import torch
    from safetensors import safe_open

    files = {p.name: (p.read_bytes() if p.suffix == ".bin" else p.read_text()) for p in sorted(ckpt_dir.iterdir())
             if p.is_file() and SIDECAR_FILE.match(p.name)}
    rng = {}
    for p in sorted(ckpt_dir.glob("rng.rank_*.pt")):
        blob = torch.load(p, map_location="cpu", weights_only=True)
        rng[int(p.stem.rsplit("_", 1)[1])] = {"cpu": blob["cpu"], "cuda": blob.get("cuda")}
    grads = None
    if (ckpt_dir / GRADIENTS).is_file():
        with safe_open(str(ckpt_dir / GRADIENTS), framework="pt") as f:
            grads = {"tensors": {k: f.get_tensor(k) for k in f.keys()}, "metadata": dict(f.metadata() or {})}
    return {"files": files, "rng": rng, "grads": grads} if (files or rng or grads is not None) else None


def check_sidecar(sc: Any) -> dict:
    """A sidecar decoded from an untrusted header, before any of it reaches the disk."""
    import torch

    def bad(why):
        raise ConversionError("refusing the file's sidecar: %s" % why)

    if not isinstance(sc, dict) or set(sc) != {"files", "rng", "grads"} or not isinstance(sc["files"], dict) or not isinstance(sc["rng"], dict):
        bad("it is not {files, rng, grads}")
    for name, content in sc["files"].items():
        if not isinstance(name, str) or not SIDECAR_FILE.match(name):
            bad("%r is not a checkpoint file name (names become paths)" % (name,))
        if not isinstance(content, (str, bytes)):
            bad("%s is neither text nor bytes" % name)
    for rank, blob in sc["rng"].items():
        if isinstance(rank, bool) or not isinstance(rank, int) or rank < 0:
            bad("RNG rank %r" % (rank,))
        if not isinstance(blob, dict) or set(blob) != {"cpu", "cuda"} or not isinstance(blob["cpu"], torch.Tensor):
            bad("RNG state of rank %d" % rank)
        cuda = blob["cuda"]
        if not (cuda is None or isinstance(cuda, torch.Tensor) or (isinstance(cuda, list) and all(isinstance(t, torch.Tensor) for t in cuda))):
            bad("CUDA RNG state of rank %d" % rank)
    g = sc["grads"]
    if g is not None:
        ok = (isinstance(g, dict) and set(g) == {"tensors", "metadata"} and isinstance(g["tensors"], dict) and isinstance(g["metadata"], dict)
              and all(isinstance(k, str) and isinstance(t, torch.Tensor) for k, t in g["tensors"].items())
              and all(isinstance(k, str) and isinstance(v, str) for k, v in g["metadata"].items()))
        if not ok:
            bad("the gradient entry")
    return sc


def write_sidecar(ckpt_dir: Path, sc: dict) -> None:
    import torch
    from safetensors.torch import save_file

    from ..train.checkpoint import COMPLETE

    for name, content in sc["files"].items():
        if isinstance(content, bytes):
            (ckpt_dir / name).write_bytes(content)
        else:
            (ckpt_dir / name).write_text(content)
    for rank, blob in sc["rng"].items():
        torch.save({"cpu": blob["cpu"], "cuda": blob["cuda"]}, ckpt_dir / ("rng.rank_%d.pt" % rank))
    if sc["grads"] is not None:
        save_file({k: t.contiguous() for k, t in sc["grads"]["tensors"].items()}, str(ckpt_dir / GRADIENTS), metadata=sc["grads"]["metadata"] or None)
    (ckpt_dir / COMPLETE).write_text("")


# ------------------------------------------------------------------------------------------------------ conversions
def to_safetensors(ckpt_path: str | Path, out_file: str | Path, keys: list[str] | None = None, verify: bool = False) -> dict:
    from safetensors import safe_open
    from safetensors.torch import save_file

    ckpt_path, out_file = Path(ckpt_path), Path(out_file)
    dcp_dir = resolve_dcp_dir(ckpt_path)
    state = read_dcp(dcp_dir)
    if keys:
        absent = [k for k in keys if k not in state]
        if absent:
            raise ConversionError("--keys %s: not in the checkpoint, whose top-level keys are %s" % (absent, sorted(state)))
        state = {k: state[k] for k in keys}
    enc = _Encoder()
    skeleton = enc.encode(state)
    header = {FORMAT_KEY: FORMAT, SKELETON_KEY: json.dumps(skeleton, separators=(",", ":"))}
    sidecar = collect_sidecar(dcp_dir.parent) if (not keys and dcp_dir.name == "dcp") else None
    if sidecar is not None:
        header[SIDECAR_KEY] = json.dumps(enc.encode(sidecar, ("__sidecar__",)), separators=(",", ":"))
    out_file.parent.mkdir(parents=True, exist_ok=True)
    save_file(enc.tensors, str(out_file), metadata=header)
    if verify:
        with safe_open(str(out_file), framework="pt") as f:
            back = f.metadata() or {}
            if json.loads(back.get(SKELETON_KEY, "null")) != skeleton:
                raise ConversionError("verify FAILED: the skeleton read back from %s differs" % out_file)
            on_disk = set(f.keys())
            if on_disk != set(enc.tensors):
                raise ConversionError("verify FAILED: tensor names differ (file only: %s; memory only: %s)"
                                      % (sorted(on_disk - set(enc.tensors))[:5], sorted(set(enc.tensors) - on_disk)[:5]))
            for k, t in enc.tensors.items():
                if not same_bits(f.get_tensor(k), t):
                    raise ConversionError("verify FAILED: tensor %r differs in %s" % (k, out_file))
    return {"file": str(out_file), "tensors": len(enc.tensors), "bytes": sum(t.numel() * t.element_size() for t in enc.tensors.values()),
            "top_level_keys": sorted(state), "sidecar_files": None if sidecar is None else sorted(sidecar["files"]) + ["rng.rank_%d.pt" % r for r in sorted(sidecar["rng"])],
            "verified": bool(verify)}


def from_safetensors(in_file: str | Path, out_dir: str | Path, top_level_key: str | None = None, verify: bool = False) -> dict:
    from safetensors import safe_open

    in_file, out_dir = Path(in_file), Path(out_dir)
    with safe_open(str(in_file), framework="pt") as f:
        header = f.metadata() or {}
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    sidecar = None
    if SKELETON_KEY in header:
        if header.get(FORMAT_KEY) != FORMAT:
            raise ConversionError("%s: %s=%r, expected %r" % (in_file, FORMAT_KEY, header.get(FORMAT_KEY), FORMAT))
        if top_level_key is not None:
            raise ConversionError("--top-level-key is for foreign files; this one carries its own structure")
        skeleton = json.loads(header[SKELETON_KEY])
        state = decode(skeleton, tensors)
        if SIDECAR_KEY in header:
            sidecar = check_sidecar(decode(json.loads(header[SIDECAR_KEY]), tensors))
    else:
        state = {top_level_key: tensors} if top_level_key else dict(tensors)
    if out_dir.exists() and any(out_dir.iterdir()):
        raise ConversionError("refusing to write into the non-empty %s (a DCP writer adds files, it does not replace a checkpoint)" % out_dir)
    target = out_dir / "dcp" if sidecar is not None else out_dir
    target.mkdir(parents=True, exist_ok=True)
    write_dcp(state, target)
    if sidecar is not None:
        write_sidecar(out_dir, sidecar)
    if verify:
        if not same_state(state, read_dcp(target)):
            raise ConversionError("verify FAILED: the state re-read from %s differs from the one decoded from %s" % (target, in_file))
        if sidecar is not None and not same_state(sidecar, collect_sidecar(out_dir)):
            raise ConversionError("verify FAILED: the sidecar re-read from %s differs from the one decoded from %s" % (out_dir, in_file))
    return {"dir": str(out_dir), "tensors": len(tensors), "top_level_keys": sorted(map(str, state)),
            "sidecar_files": None if sidecar is None else sorted(sidecar["files"]) + ["rng.rank_%d.pt" % r for r in sorted(sidecar["rng"])],
            "verified": bool(verify)}


def pack(ckpt_dir: str, out_file: str, verify: bool = False) -> dict:
    """A complete ``step_N`` directory -> one file (tensors + resume sidecar)."""
    from ..train.checkpoint import COMPLETE

    if not (Path(ckpt_dir) / COMPLETE).exists():
        raise FileNotFoundError("%s is not a complete checkpoint" % ckpt_dir)
    return to_safetensors(ckpt_dir, out_file, verify=verify)


def unpack(in_file: str, out_dir: str, verify: bool = False) -> dict:
    return from_safetensors(in_file, out_dir, verify=verify)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pretrain-dcp-safetensors", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("to-safetensors", aliases=["pack"], help="DCP checkpoint -> one .safetensors file")
    t.add_argument("checkpoint", type=Path, help="step_N directory (with dcp/ inside) or the DCP directory itself")
    t.add_argument("output", type=Path)
    t.add_argument("--keys", nargs="+", default=None, metavar="KEY", help="only these top-level keys, e.g. `--keys model` (tensors only, no sidecar)")
    t.add_argument("--verify", action="store_true", help="re-read the written file and compare every tensor bit for bit")
    f = sub.add_parser("from-safetensors", aliases=["unpack"], help=".safetensors file -> DCP checkpoint")
    f.add_argument("input", type=Path)
    f.add_argument("output", type=Path, help="created; must be empty: a step_N directory when the file carries a sidecar, else a bare DCP directory")
    f.add_argument("--top-level-key", default=None, metavar="KEY", help="nest a foreign file's tensors under this key, e.g. `model`")
    f.add_argument("--verify", action="store_true", help="re-read the written checkpoint offline and compare bit for bit")
    a = ap.parse_args(argv)
    try:
        if a.cmd in ("to-safetensors", "pack"):
            res = to_safetensors(a.checkpoint, a.output, keys=a.keys, verify=a.verify)
        else:
            res = from_safetensors(a.input, a.output, top_level_key=a.top_level_key, verify=a.verify)
    except ConversionError as e:
        print("pretrain-dcp-safetensors: %s" % e, file=sys.stderr)
        return 2
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
