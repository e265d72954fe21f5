"""Checkpoint directory: writer, reader, metadata, integrity gates.

Layout of ``<run>/checkpoints/step_%09d/`` (reference src/pretrain/train/checkpoint.py:271-326, 743-782)::

    dcp/                       torch.distributed.checkpoint of {"model": {name: fp32 tensor}, "optim": {"state": {index:
                               {"step", "exp_avg", "exp_avg_sq"}}, "param_groups": [{..., "params": [indices]}]}} - the payload
                               of `model.state_dict()` / `optimizer.state_dict()` (parameters numbered group by group, in
                               `named_parameters()` order inside a group), as the reference saves it
    meta.json                  CheckpointMeta
    state_hash.txt             hash of the state at this step (hex)
    global_stream.json         position of the canonical data stream (same on every rank)
    spike_protocol.json        spike / cool-down state
    rng.rank_<v>.pt            {"cpu": ByteTensor, "cuda": ByteTensor | None} per virtual rank
    batch_hasher.rank_<v>.bin  32-byte running batch digest per virtual rank
    _COMPLETE                  written last; a directory without it is ignored

Every process writes the rows of the tensors it owns into ``dcp/`` (a distributed DCP save over a dedicated gloo
group: one data file per process, metadata committed by rank 0; reference src/pretrain/train/checkpoint.py:589-627),
from a snapshot in pinned host memory taken when ``save`` is called, so the writing can run on a background thread
while training goes on. Rank 0 writes every small file (reference :724-741) and, last, ``_COMPLETE``. Reading never
unpickles untrusted code: the DCP ``.metadata`` pickle goes through an allow-listing unpickler first and ``.pt``
files are loaded with ``weights_only=True``. Checkpoints whose optimizer state is keyed by parameter name (written
by earlier versions of this package) still load.
"""
from __future__ import annotations

import dataclasses
import io
import json
import pickle
import re
import shutil
import threading
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
    replicate_reduce_algo: str = "recursive_doubling"   # parallel/deterministic_reduce.py::REPLICATE_REDUCE_ALGO
    grad_norm_algo: str = "deterministic_per_tensor_sos_v1"
    clip_algo: str = "global"
    tensor_digest: str = "raw"
    rewarm_anchor_tokens: int | None = None
    seed: int = 0
    torch_version: str = ""
    numpy_version: str = ""
    kernel_env: dict = dataclasses.field(default_factory=dict)
    # REPOP_* variables of the writing process: the reference's meta.json field of that name (its kernel library's switches);
    # this package's own switches are `kernel_env`
    repop_env: dict = dataclasses.field(default_factory=dict)
    native_source_digests: dict = dataclasses.field(default_factory=dict)   # sha256 of each native library's sources + flags
    windows_emitted: int = 0
    physical_world_size: int = 1
    mixed_precision: bool = True
    optimizer_param_names: list = dataclasses.field(default_factory=list)   # parameter name of optim.state.<index>, by index

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
class OwnedRows:
    """One tensor of the checkpoint as THIS process holds it: the global shape and dtype, and the row ranges it owns as
    (first row, CPU tensor of those rows). The planner below turns every piece into one DCP chunk."""

    def __init__(self, shape, dtype, pieces):
        self.shape, self.dtype, self.pieces = tuple(shape), dtype, list(pieces)


def _save_planner():
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
    from torch.distributed.checkpoint.planner import SavePlan, TensorWriteData, WriteItem, WriteItemType
    from torch.distributed.checkpoint.planner_helpers import _create_write_items

    class OwnedRowsPlanner(dcp.DefaultSavePlanner):
        """Sharded tensors arrive as `OwnedRows`: each owned row range becomes a SHARD write item at its offset in the
        global tensor, so the chunks of all processes tile the tensor and any reader can re-shard them. Everything that
        is the same on every process (step counters, param_groups) is written by the coordinator alone."""

        def create_local_plan(self):
            items = []
            for fqn, obj in self.state_dict.items():
                if isinstance(obj, OwnedRows):
                    rest = [0] * (len(obj.shape) - 1)
                    for row_lo, t in obj.pieces:
                        offs = torch.Size([row_lo] + rest) if obj.shape else torch.Size([])
                        props = TensorProperties(dtype=obj.dtype)
                        items.append(WriteItem(index=MetadataIndex(fqn, offs), type=WriteItemType.SHARD,
                                               tensor_data=TensorWriteData(chunk=ChunkStorageMetadata(offsets=offs, sizes=t.shape),
                                                                           properties=props, size=torch.Size(obj.shape))))
                elif self.is_coordinator:
                    items += _create_write_items(fqn, obj)
            plan = SavePlan(items)
            if self.flatten_state_dict:
                plan = dataclasses.replace(plan, planner_data=self.mappings)
            self.plan = plan
            return plan

        def lookup_object(self, index):
            obj = self.state_dict[index.fqn]
            if isinstance(obj, OwnedRows):
                for row_lo, t in obj.pieces:
                    if not obj.shape or row_lo == index.offset[0]:
                        return t
                raise KeyError("no piece of %s at %s" % (index.fqn, tuple(index.offset)))
            return super().lookup_object(index)

    return OwnedRowsPlanner()


def optimizer_param_indices(param_groups, names, members) -> dict[str, int]:
    """Parameter name -> index in `optimizer.state_dict()`: parameters are numbered group by group, inside a group in
    `named_parameters()` order (what torch.optim.Optimizer.state_dict does with the groups of optim/adamw.py)."""
    out, nxt = {}, 0
    for gi in range(len(param_groups)):
        for n, m in zip(names, members):
            if m == gi:
                out[n] = nxt
                nxt += 1
    return out


class Checkpointer:
    def __init__(self, run_dir: str | Path, rank: int = 0, world: int = 1, group=None):
        self.root = Path(run_dir) / "checkpoints"
        self.rank, self.world, self.group = rank, world, group
        self._writer: threading.Thread | None = None
        self._writer_error: list = []
        self._pinned: dict = {}
        self._save_group = None
        if world > 1:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                # DCP's planning collectives and the commit barrier run on their own gloo group, possibly from a background
                # thread, and never interleave with the training collectives (reference src/pretrain/train/checkpoint.py:259-269)
                self._save_group = dist.new_group(backend="gloo")

    def step_dir(self, step: int) -> Path:
        return self.root / ("step_%09d" % step)

    # -- save -------------------------------------------------------------------------------------------
    def save(self, step: int, engine, meta: CheckpointMeta, state_hash: str | None, stream_state: dict | None,
             spike_state: dict | None, batch_chains: dict[int, bytes], rng_states: dict[int, dict] | None = None,
             wait: bool = True) -> Path:
        """``batch_chains`` / ``rng_states`` map VIRTUAL rank -> payload for the ranks this process hosts; they are
        gathered to rank 0, which writes the small files. The tensors are snapshotted here (device -> pinned host memory)
        and written by every owner; with ``wait=False`` the writing, the commit barrier and ``_COMPLETE`` happen on a
        background thread and ``wait()`` (or the next ``save``) joins it."""
        import torch.distributed as dist

        self.wait()
        t0 = time.time()
        d = self.step_dir(step)
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
            for v in range(meta.dp_world_size):
                if v not in chains:
                    raise FileNotFoundError("no batch-hasher chain for virtual rank %d" % v)
                (d / ("batch_hasher.rank_%d.bin" % v)).write_bytes(chains[v])
                rng = rngs.get(v) or {"cpu": torch.get_rng_state(), "cuda": None}
                torch.save(rng, d / ("rng.rank_%d.pt" % v))
            if stream_state is not None:
                (d / "global_stream.json").write_text(json.dumps(stream_state))
            (d / "spike_protocol.json").write_text(json.dumps(spike_state or {}))
            index = optimizer_param_indices(engine.param_groups, engine.layout.names, engine.layout.groups)
            meta = dataclasses.replace(meta, optimizer_param_names=sorted(index, key=index.get))
            (d / "meta.json").write_text(meta.to_json())
            (d / "dcp").mkdir(parents=True, exist_ok=True)
        if self.world > 1:
            dist.barrier(group=self._save_group)  # the directory exists before anyone writes into it
        state = self._snapshot(engine)
        self.last_snapshot_s = time.time() - t0

        def write():
            try:
                self._write_tensors(d / "dcp", state)
                if self.world > 1:
                    dist.barrier(group=self._save_group)
                if self.rank == 0:
                    (d / COMPLETE).write_text("%.3f\n" % (time.time() - t0))
            except BaseException as e:  # surfaces in wait()
                self._writer_error.append(e)

        if wait:
            write()
            self.wait()
        else:
            self._writer = threading.Thread(target=write, name="checkpoint-writer", daemon=True)
            self._writer.start()
        return d

    def wait(self) -> None:
        """Block until a background save has been committed; raises what the writer raised."""
        if self._writer is not None:
            self._writer.join()
            self._writer = None
        if self._writer_error:
            raise self._writer_error.pop()

    def _stage(self, key: str, count: int, dtype, device_is_cuda: bool) -> torch.Tensor:
        buf = self._pinned.get(key)
        if buf is None or buf.numel() < count or buf.dtype != dtype:
            buf = torch.empty(max(count, 1), dtype=dtype, pin_memory=device_is_cuda)
            self._pinned[key] = buf
        return buf

    def prepare(self, engine) -> None:
        """Allocate (page-lock) the host staging buffers of this process's rows now, so that the first checkpoint of a run
        does not pay for it on the training thread (page-locking runs at 1-2 GB/s: 11 s for the 19 GB of one GPU holding
        everything, 2.5 s per process on eight)."""
        if not engine.is_cuda:
            return
        total = sum(t["weight"].numel() for pp in engine.owned_pieces() for _lo, _hi, t in pp)
        for k in ("weight", "exp_avg", "exp_avg_sq"):
            self._stage(k, total, torch.float32, True)

    def _snapshot(self, engine) -> dict:
        """This process's rows of master weights and moments, copied to (pinned) host memory, in the reference's layout."""
        lay = engine.layout
        owned = engine.owned_pieces()
        index = optimizer_param_indices(engine.param_groups, lay.names, lay.groups)
        is_cuda = engine.is_cuda
        total = sum(t["weight"].numel() for pp in owned for _lo, _hi, t in pp)
        kinds = ("weight", "exp_avg", "exp_avg_sq")
        stage = {k: self._stage(k, total, torch.float32, is_cuda) for k in kinds}
        pieces = {k: [[] for _ in lay.names] for k in kinds}
        off = 0
        for i, pp in enumerate(owned):
            shape = lay.shapes[i]
            for lo, hi, tensors in pp:
                n = tensors["weight"].numel()
                for k in kinds:
                    dst = stage[k][off:off + n]
                    dst.copy_(tensors[k], non_blocking=is_cuda)
                    pieces[k][i].append((lo, dst.view((hi - lo,) + tuple(shape[1:])) if shape else dst.view(())))
                off += n
        if is_cuda:
            torch.cuda.current_stream().synchronize()
        model = {n: OwnedRows(lay.shapes[i], torch.float32, pieces["weight"][i]) for i, n in enumerate(lay.names)}
        state = {index[n]: {"step": torch.tensor(int(engine.opt_step), dtype=torch.int64),
                            "exp_avg": OwnedRows(lay.shapes[i], torch.float32, pieces["exp_avg"][i]),
                            "exp_avg_sq": OwnedRows(lay.shapes[i], torch.float32, pieces["exp_avg_sq"][i])} for i, n in enumerate(lay.names)}
        groups = []
        for gi, g in enumerate(engine.param_groups):
            groups.append(dict(g, params=[index[n] for n, m in zip(lay.names, lay.groups) if m == gi]))
        return {"model": model, "optim": {"state": state, "param_groups": groups}}

    def _write_tensors(self, dcp_dir: Path, state: dict) -> None:
        import torch.distributed.checkpoint as dcp

        dcp.save(state, storage_writer=dcp.FileSystemWriter(str(dcp_dir), thread_count=4, sync_files=False), planner=_save_planner(),
                 process_group=self._save_group, no_dist=self.world == 1)

    @staticmethod
    def _template(engine, keyed_by_name: bool, load_optimizer: bool) -> dict:
        lay = engine.layout
        model = {n: torch.empty(lay.shapes[i], dtype=torch.float32) for i, n in enumerate(lay.names)}
        if not load_optimizer:
            return {"model": model}
        index = optimizer_param_indices(engine.param_groups, lay.names, lay.groups)
        key = (lambda n: n) if keyed_by_name else (lambda n: index[n])
        st = {key(n): {"step": torch.zeros((), dtype=torch.int64), "exp_avg": torch.empty(lay.shapes[i], dtype=torch.float32),
                       "exp_avg_sq": torch.empty(lay.shapes[i], dtype=torch.float32)} for i, n in enumerate(lay.names)}
        groups = [dict(g) if keyed_by_name else dict(g, params=[index[n] for n, m in zip(lay.names, lay.groups) if m == gi])
                  for gi, g in enumerate(engine.param_groups)]
        return {"model": model, "optim": {"state": st, "param_groups": groups}}

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
        reader = dcp.FileSystemReader(str(d / "dcp"))
        keyed_by_name = not any(k.startswith("optim.state.0.") for k in reader.read_metadata().state_dict_metadata)
        template = self._template(engine, keyed_by_name, load_optimizer)
        dcp.load(template, storage_reader=dcp.FileSystemReader(str(d / "dcp")), no_dist=True)
        lay = engine.layout
        index = optimizer_param_indices(engine.param_groups, lay.names, lay.groups)
        key = (lambda n: n) if keyed_by_name else (lambda n: index[n])
        for i, n in enumerate(engine.names):
            st = template["optim"]["state"][key(n)] if load_optimizer else None
            engine.load_parameter_state(i, template["model"][n], st["exp_avg"] if st else None, st["exp_avg_sq"] if st else None)
        if load_optimizer:
            steps = {int(template["optim"]["state"][key(n)]["step"]) for n in engine.names}
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


def optimizer_state_names(ckpt_dir: str | Path) -> dict[str, str]:
    """`optim.state.<key>` -> parameter name for a checkpoint directory: the index list recorded in meta.json for the
    torch-style payload; empty for checkpoints whose optimizer state is keyed by name already."""
    p = Path(ckpt_dir) / "meta.json"
    if not p.is_file():
        return {}
    names = json.loads(p.read_text()).get("optimizer_param_names") or []
    return {str(i): n for i, n in enumerate(names)}


def resolved_config_json(cfg) -> str:
    return json.dumps(cfg.model_dump(mode="json"), sort_keys=True)
