"""Checkpoint directory: writer, reader, metadata, integrity gates.

Layout of ``<run>/checkpoints/step_%09d/`` (reference src/pretrain/train/checkpoint.py:271-326, 743-782)::

    dcp/                       torch.distributed.checkpoint of {"model": {name: fp32 tensor}, "optim": {"state": {name:
                               {"step", "exp_avg", "exp_avg_sq"}}, "param_groups": [...]}}
    meta.json                  CheckpointMeta
    state_hash.txt             hash of the state at this step (hex)
    global_stream.json         position of the canonical data stream (same on every rank)
    spike_protocol.json        spike / cool-down state
    rng.rank_<v>.pt            {"cpu": ByteTensor, "cuda": ByteTensor | None} per virtual rank
    batch_hasher.rank_<v>.bin  32-byte running batch digest per virtual rank
    _COMPLETE                  written last; a directory without it is ignored

Rank 0 writes every file (after the engine gathered the full state), so a lossy shared filesystem sees
one writer. Reading never unpickles untrusted code: the DCP ``.metadata`` pickle goes through an
allow-listing unpickler first and ``.pt`` files are loaded with ``weights_only=True``.
"""
from __future__ import annotations

import dataclasses
import io
import json
import pickle
import re
import shutil
import time
from pathlib import Path
from typing import Any

import torch

COMPLETE = "_COMPLETE"
STEP_DIR = re.compile(r"^step_(\d{9})$")


@dataclasses.dataclass
class CheckpointMeta:
    consumed_tokens: int = 0
    step: int = 0
    git_sha: str = ""
    config_resolved: str = ""          # JSON of the fully resolved config
    tokenizer_hash: str = ""
    container_digest: str = ""
    restart_count: int = 0
    chained_hash: str | None = None    # running chain (advanced only on cadence steps)
    reduction_mode: str = "deterministic_allgather"
    dp_world_size: int = 1             # VIRTUAL data-parallel world size
    dp_replicate: int = 1
    dp_shard: int = 1
    replicate_reduce_algo: str = "binary_blocks_tree"
    grad_norm_algo: str = "deterministic_per_tensor_sos_v1"
    clip_algo: str = "global"
    tensor_digest: str = "raw"
    rewarm_anchor_tokens: int | None = None
    seed: int = 0
    torch_version: str = ""
    numpy_version: str = ""
    kernel_env: dict = dataclasses.field(default_factory=dict)
    native_source_digests: dict = dataclasses.field(default_factory=dict)   # sha256 of each native library's sources + flags
    windows_emitted: int = 0
    physical_world_size: int = 1
    mixed_precision: bool = True

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1, sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "CheckpointMeta":
        d = json.loads(text)
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


# ------------------------------------------------------------------ untrusted-pickle gate for DCP metadata
_ALLOWED_PREFIXES = ("torch.distributed.checkpoint.metadata", "torch.distributed.checkpoint.", "collections", "builtins")
_ALLOWED_EXACT = {("torch", "Size"), ("torch", "dtype"), ("torch._utils", "_rebuild_tensor_v2"), ("torch", "device"),
                  ("torch.serialization", "_get_layout"), ("torch", "memory_format"), ("pathlib", "PosixPath"), ("pathlib", "PurePosixPath"),
                  ("pathlib", "Path"), ("pathlib._local", "PosixPath"), ("pathlib._local", "PurePosixPath")}
_BUILTINS_OK = {"dict", "list", "tuple", "set", "frozenset", "int", "float", "str", "bytes", "bool", "complex", "slice", "range", "object",
                "getattr_not_allowed"}


class UntrustedCheckpointError(RuntimeError):
    pass


class _AllowListUnpickler(pickle.Unpickler):
    def find_class(self, module: str, name: str):
        if module == "builtins":
            if name in _BUILTINS_OK and name != "getattr_not_allowed":
                return super().find_class(module, name)
            raise UntrustedCheckpointError("checkpoint metadata references builtins.%s" % name)
        if (module, name) in _ALLOWED_EXACT:
            return super().find_class(module, name)
        if module.startswith("torch.distributed.checkpoint") or module in ("collections",):
            return super().find_class(module, name)
        if module == "torch" and (name.endswith("Storage") or
                                  isinstance(getattr(torch, name, None), (torch.dtype, torch.layout, torch.memory_format))):
            return super().find_class(module, name)
        raise UntrustedCheckpointError("checkpoint metadata references %s.%s, which is not on the allow-list" % (module, name))


def validate_dcp_metadata(dcp_dir: str | Path) -> None:
    """Parse ``dcp/.metadata`` with the allow-listing unpickler; raises before anything dangerous can run."""
    p = Path(dcp_dir) / ".metadata"
    if not p.is_file():
        raise FileNotFoundError("%s missing" % p)
    try:
        _AllowListUnpickler(io.BytesIO(p.read_bytes())).load()
    except UntrustedCheckpointError:
        raise
    except Exception as e:  # malformed pickle
        raise UntrustedCheckpointError("cannot parse %s safely: %r" % (p, e))


# ------------------------------------------------------------------------------------------ writer / reader
class Checkpointer:
    def __init__(self, run_dir: str | Path, rank: int = 0, world: int = 1, group=None):
        self.root = Path(run_dir) / "checkpoints"
        self.rank, self.world, self.group = rank, world, group

    def step_dir(self, step: int) -> Path:
        return self.root / ("step_%09d" % step)

    # -- save -------------------------------------------------------------------------------------------
    def save(self, step: int, engine, meta: CheckpointMeta, state_hash: str | None, stream_state: dict | None,
             spike_state: dict | None, batch_chains: dict[int, bytes], rng_states: dict[int, dict] | None = None) -> Path:
        """``batch_chains`` / ``rng_states`` map VIRTUAL rank -> payload for the ranks this process hosts; they are
        gathered to rank 0, which writes everything."""
        import torch.distributed as dist

        t0 = time.time()
        d = self.step_dir(step)
        engine.gather_full_state()
        chains, rngs = dict(batch_chains), dict(rng_states or {})
        if self.world > 1:
            objs: list = [None] * self.world
            dist.all_gather_object(objs, (chains, rngs), group=self.group)
            chains = {k: v for c, _ in objs for k, v in c.items()}
            rngs = {k: v for _, r in objs for k, v in r.items()}
        if self.rank == 0:
            if d.exists():
                shutil.rmtree(d)
            d.mkdir(parents=True)
            if state_hash is not None:
                (d / "state_hash.txt").write_text(state_hash + "\n")
            self._write_tensors(d / "dcp", engine)
            for v in range(meta.dp_world_size):
                if v not in chains:
                    raise FileNotFoundError("no batch-hasher chain for virtual rank %d" % v)
                (d / ("batch_hasher.rank_%d.bin" % v)).write_bytes(chains[v])
                rng = rngs.get(v) or {"cpu": torch.get_rng_state(), "cuda": None}
                torch.save(rng, d / ("rng.rank_%d.pt" % v))
            if stream_state is not None:
                (d / "global_stream.json").write_text(json.dumps(stream_state))
            (d / "spike_protocol.json").write_text(json.dumps(spike_state or {}))
            (d / "meta.json").write_text(meta.to_json())
            (d / COMPLETE).write_text("%.3f\n" % (time.time() - t0))
        if self.world > 1:
            dist.barrier(group=self.group)
        return d

    @staticmethod
    def _state_dict(engine) -> dict:
        model = {n: t.detach().to("cpu").clone() for n, t in engine.named_master()}
        optim_state = {n: {"step": torch.tensor(int(st["step"]), dtype=torch.int64), "exp_avg": st["exp_avg"].detach().to("cpu").clone(),
                           "exp_avg_sq": st["exp_avg_sq"].detach().to("cpu").clone()} for n, st in engine.optimizer_state().items()}
        return {"model": model, "optim": {"state": optim_state, "param_groups": [dict(g) for g in engine.param_groups]}}

    def _write_tensors(self, dcp_dir: Path, engine) -> None:
        import torch.distributed.checkpoint as dcp

        dcp_dir.mkdir(parents=True, exist_ok=True)
        dcp.save(self._state_dict(engine), storage_writer=dcp.FileSystemWriter(str(dcp_dir), thread_count=1), no_dist=True)

    # -- load -------------------------------------------------------------------------------------------
    @staticmethod
    def read_meta(ckpt_dir: str | Path) -> CheckpointMeta:
        return CheckpointMeta.from_json((Path(ckpt_dir) / "meta.json").read_text())

    def load(self, ckpt_dir: str | Path, engine, load_optimizer: bool = True) -> dict:
        """Restore weights (+ optimizer) into ``engine``; returns the side files as a dict."""
        import torch.distributed.checkpoint as dcp

        d = Path(ckpt_dir)
        if not (d / COMPLETE).exists():
            raise FileNotFoundError("%s has no %s marker (incomplete checkpoint)" % (d, COMPLETE))
        meta = self.read_meta(d)
        validate_dcp_metadata(d / "dcp")
        template = self._state_dict(engine)
        if not load_optimizer:
            template = {"model": template["model"]}
        dcp.load(template, storage_reader=dcp.FileSystemReader(str(d / "dcp")), no_dist=True)
        lay = engine.layout
        with torch.no_grad():
            for i, n in enumerate(engine.names):
                lay.view(engine.master, i).copy_(template["model"][n])
                if load_optimizer:
                    st = template["optim"]["state"][n]
                    lay.view(engine.m1, i).copy_(st["exp_avg"])
                    lay.view(engine.m2, i).copy_(st["exp_avg_sq"])
        if load_optimizer:
            steps = {int(template["optim"]["state"][n]["step"]) for n in engine.names}
            if len(steps) != 1:
                raise ValueError("parameters disagree on the optimizer step: %s" % sorted(steps))
            engine.opt_step = steps.pop()
            for g, saved in zip(engine.param_groups, template["optim"]["param_groups"]):
                g.update({k: v for k, v in saved.items() if k != "params"})
        engine.refresh_compute_weights()
        side: dict[str, Any] = {"meta": meta}
        side["state_hash"] = (d / "state_hash.txt").read_text().strip() if (d / "state_hash.txt").exists() else None
        side["global_stream"] = json.loads((d / "global_stream.json").read_text()) if (d / "global_stream.json").exists() else None
        side["spike_protocol"] = json.loads((d / "spike_protocol.json").read_text()) if (d / "spike_protocol.json").exists() else {}
        chains, rngs = {}, {}
        for v in range(meta.dp_world_size):
            p = d / ("batch_hasher.rank_%d.bin" % v)
            if not p.exists():
                raise FileNotFoundError("checkpoint %s lacks %s" % (d, p.name))
            chains[v] = p.read_bytes()
            r = d / ("rng.rank_%d.pt" % v)
            if not r.exists():
                raise FileNotFoundError("checkpoint %s lacks %s" % (d, r.name))
            rngs[v] = torch.load(r, weights_only=True)
        side["batch_chains"], side["rng"] = chains, rngs
        return side

    # -- housekeeping -------------------------------------------------------------------------------------
    def complete_steps(self) -> list[int]:
        if not self.root.is_dir():
            return []
        out = []
        for p in self.root.iterdir():
            m = STEP_DIR.match(p.name)
            if m and (p / COMPLETE).exists():
                out.append(int(m.group(1)))
        return sorted(out)

    def latest(self) -> Path | None:
        steps = self.complete_steps()
        return self.step_dir(steps[-1]) if steps else None

    def garbage_collect(self, keep_last: int = 4, keep_every: int = 10) -> list[Path]:
        """Delete complete checkpoints except the ``keep_last`` newest and every ``keep_every``-th (by order)."""
        steps = self.complete_steps()
        keep = set(steps[-keep_last:]) | {s for i, s in enumerate(steps) if keep_every and i % keep_every == 0}
        gone = []
        if self.rank == 0:
            for s in steps:
                if s not in keep:
                    shutil.rmtree(self.step_dir(s))
                    gone.append(self.step_dir(s))
        return gone


def resolved_config_json(cfg) -> str:
    return json.dumps(cfg.model_dump(mode="json"), sort_keys=True)
