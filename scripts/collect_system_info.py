#!/usr/bin/env python3
"""One JSON record of the machine a rank runs on, for a run's reproducibility file.

    python scripts/collect_system_info.py --output runs/<run_id>/system_info/pod-<index>.json [--git-path REPO ...]

Sections: ``host`` (OS, kernel, container hints), ``kubernetes`` (pod / job variables), ``cpu``, ``memory``, ``disk``,
``network`` (interfaces and addresses), ``gpu`` (inventory, clocks and limits as READ, NVLink topology), ``nvidia_driver``,
``cuda`` (toolkit, runtime, cuDNN, NCCL), ``python``, ``torch`` (build flags, determinism switches), ``kernels`` (this
package's native libraries and the digests of their sources), ``git`` (HEAD, branch, dirty flag per repository), ``env``
(variables that steer determinism, NCCL, rendezvous or kernel selection; anything that looks like a secret is redacted) and
``pip_freeze``. Every probe stands alone: a missing tool or file puts ``{"error": ...}`` into its section and the rest
goes on. The script only reads; it changes no clock, limit or mode.
(reference scripts/collect_system_info.py:99-405)
"""
from __future__ import annotations

import argparse
import json
import os
import platform
import shutil
import socket
import subprocess
import sys
from datetime import datetime, timezone
from pathlib import Path

SCHEMA_VERSION = 1
SECRET_WORDS = ("KEY", "TOKEN", "SECRET", "PASSWORD", "PASSWD", "CREDENTIAL")
ENV_PREFIXES = ("NCCL_", "TORCH_", "TORCHELASTIC_", "CUDA", "CUDNN_", "CUBLAS", "OTB_", "PRETRAIN_", "REPOP_", "HF_", "OMP_", "MKL_", "PYTHON",
                "JOB_", "POD_", "KUBERNETES_", "RUN_", "WANDB_", "MASTER_", "RDZV_", "GROUP_", "LD_LIBRARY", "LD_PRELOAD", "DIST_")
ENV_NAMES = ("HOSTNAME", "USER", "PATH", "PWD", "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "NVIDIA_VISIBLE_DEVICES",
             "NVIDIA_DRIVER_CAPABILITIES", "TF32_OVERRIDE", "CONTAINER_DIGEST")
GPU_FIELDS = ("index", "name", "uuid", "driver_version", "vbios_version", "memory.total", "memory.used", "clocks.sm", "clocks.max.sm",
              "clocks.mem", "clocks.max.mem", "power.draw", "power.limit", "temperature.gpu", "persistence_mode", "compute_mode",
              "ecc.mode.current", "mig.mode.current", "pcie.link.gen.current", "pcie.link.width.current")
PROBES: dict = {}


def probe(name):
    def register(fn):
        PROBES[name] = fn
        return fn
    return register


def sh(cmd: list[str], timeout: int = 15) -> dict:
    """Run a command; never raises. {"stdout", "returncode"} or {"error"}."""
    if shutil.which(cmd[0]) is None:
        return {"error": "%s not found" % cmd[0]}
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        return {"stdout": r.stdout.strip(), "returncode": r.returncode, **({"stderr": r.stderr.strip()[-400:]} if r.returncode else {})}
    except Exception as e:  # timeout, permission, ...
        return {"error": "%s: %s" % (type(e).__name__, e)}


def read(path: str, limit: int = 65536) -> str | None:
    try:
        with open(path, "r", errors="replace") as f:
            return f.read(limit)
    except OSError:
        return None


def redact(name: str, value: str) -> str:
    return "<redacted>" if any(w in name.upper() for w in SECRET_WORDS) else value


@probe("host")
def host() -> dict:
    release = {}
    for line in (read("/etc/os-release") or "").splitlines():
        k, _, v = line.partition("=")
        if k in ("NAME", "VERSION", "ID", "VERSION_ID", "PRETTY_NAME"):
            release[k.lower()] = v.strip('"')
    return {"hostname": socket.gethostname(), "fqdn": socket.getfqdn(), "platform": platform.platform(), "kernel": platform.release(),
            "machine": platform.machine(), "os_release": release, "in_container": os.path.exists("/.dockerenv") or "kubepods" in (read("/proc/1/cgroup") or ""),
            "boot_id": (read("/proc/sys/kernel/random/boot_id") or "").strip() or None, "uptime_s": float((read("/proc/uptime") or "0").split()[0])}


@probe("kubernetes")
def kubernetes() -> dict:
    keep = ("JOB_COMPLETION_INDEX", "POD_NAME", "POD_NAMESPACE", "POD_IP", "NODE_NAME", "KUBERNETES_SERVICE_HOST")
    return {k: os.environ.get(k) for k in keep}


@probe("cpu")
def cpu() -> dict:
    info = read("/proc/cpuinfo") or ""
    models = {line.split(":", 1)[1].strip() for line in info.splitlines() if line.startswith("model name")}
    flags = next((line.split(":", 1)[1].split() for line in info.splitlines() if line.startswith("flags")), [])
    try:
        affinity = len(os.sched_getaffinity(0))
    except AttributeError:
        affinity = None
    return {"logical_cpus": os.cpu_count(), "usable_cpus": affinity, "models": sorted(models), "sockets": len({l for l in info.splitlines() if l.startswith("physical id")}) or None,
            "simd": [f for f in ("avx2", "avx512f", "avx512_bf16", "amx_bf16", "fma") if f in flags], "numa_nodes": len(list(Path("/sys/devices/system/node").glob("node[0-9]*"))) or None}


@probe("memory")
def memory() -> dict:
    fields = {}
    for line in (read("/proc/meminfo") or "").splitlines():
        k, _, v = line.partition(":")
        if k in ("MemTotal", "MemAvailable", "SwapTotal", "HugePages_Total", "Hugepagesize", "Shmem"):
            fields[k] = v.strip()
    cg = read("/sys/fs/cgroup/memory.max") or read("/sys/fs/cgroup/memory/memory.limit_in_bytes")
    return {**fields, "cgroup_limit": (cg or "").strip() or None, "shm": _usage("/dev/shm")}


def _usage(path: str) -> dict | None:
    try:
        u = shutil.disk_usage(path)
        return {"total": u.total, "used": u.used, "free": u.free}
    except OSError:
        return None


@probe("disk")
def disk() -> dict:
    mounts = {}
    for p in dict.fromkeys(["/", os.getcwd(), "/tmp", os.environ.get("RUN_OUTPUT_DIR") or "runs"]):
        if p and os.path.exists(p):
            mounts[p] = _usage(p)
    return {"usage": mounts, "mounts": [l.split()[:3] for l in (read("/proc/mounts") or "").splitlines() if l.split()[2:3] and l.split()[2] in ("nfs", "nfs4", "lustre", "ext4", "xfs", "overlay", "tmpfs", "fuse")][:40]}


@probe("network")
def network() -> dict:
    out: dict = {"interfaces": {}}
    for dev in sorted(Path("/sys/class/net").glob("*")):
        out["interfaces"][dev.name] = {"state": (read(str(dev / "operstate")) or "").strip(), "mtu": (read(str(dev / "mtu")) or "").strip(),
                                       "speed_mbps": (read(str(dev / "speed")) or "").strip() or None}
    try:
        out["addresses"] = sorted({ai[4][0] for ai in socket.getaddrinfo(socket.gethostname(), None)})
    except OSError as e:
        out["addresses"] = {"error": str(e)}
    ib = sh(["ibstat", "-l"])
    out["infiniband"] = ib.get("stdout", "").split() if "stdout" in ib else ib
    return out


@probe("gpu")
def gpu() -> dict:
    q = sh(["nvidia-smi", "--query-gpu=" + ",".join(GPU_FIELDS), "--format=csv,noheader,nounits"])
    if "stdout" not in q or q.get("returncode"):
        return {"available": False, **q}
    devices = [dict(zip(GPU_FIELDS, [c.strip() for c in line.split(",")])) for line in q["stdout"].splitlines() if line.strip()]
    return {"available": bool(devices), "count": len(devices), "devices": devices, "topology": sh(["nvidia-smi", "topo", "-m"]).get("stdout"),
            "nvlink": sh(["nvidia-smi", "nvlink", "--status"], timeout=30).get("stdout")}


@probe("nvidia_driver")
def nvidia_driver() -> dict:
    return {"proc_version": (read("/proc/driver/nvidia/version") or "").strip() or None,
            "modules": [l.split()[0] for l in (read("/proc/modules") or "").splitlines() if l.startswith(("nvidia", "gdrdrv", "nv_peer"))],
            "fabric_manager": sh(["nv-fabricmanager", "--version"]).get("stdout")}


@probe("cuda")
def cuda() -> dict:
    out = {"nvcc": (sh(["nvcc", "--version"]).get("stdout") or "").splitlines()[-2:] or None, "cuda_home": os.environ.get("CUDA_HOME") or ("/usr/local/cuda" if os.path.isdir("/usr/local/cuda") else None)}
    try:
        import torch

        out.update({"torch_cuda": torch.version.cuda, "cudnn": torch.backends.cudnn.version() if torch.backends.cudnn.is_available() else None,
                    "nccl": ".".join(map(str, torch.cuda.nccl.version())) if hasattr(torch.cuda, "nccl") and torch.cuda.is_available() else None})
    except Exception as e:
        out["torch"] = {"error": repr(e)}
    return out


@probe("python")
def python() -> dict:
    return {"version": sys.version, "executable": sys.executable, "prefix": sys.prefix, "implementation": platform.python_implementation(),
            "path_head": sys.path[:6]}


@probe("torch")
def torch_info() -> dict:
    import torch

    out = {"version": torch.__version__, "cuda_built": torch.version.cuda, "git": getattr(torch.version, "git_version", None),
           "cuda_available": torch.cuda.is_available(), "device_count": torch.cuda.device_count(), "arch_list": torch.cuda.get_arch_list() if torch.cuda.is_available() else [],
           "deterministic_algorithms": torch.are_deterministic_algorithms_enabled(), "cudnn_deterministic": torch.backends.cudnn.deterministic,
           "cudnn_benchmark": torch.backends.cudnn.benchmark, "matmul_tf32": torch.backends.cuda.matmul.allow_tf32, "cudnn_tf32": torch.backends.cudnn.allow_tf32,
           "threads": torch.get_num_threads(), "distributed_backends": {"nccl": torch.distributed.is_nccl_available(), "gloo": torch.distributed.is_gloo_available()}}
    if torch.cuda.is_available():
        out["devices"] = [{"index": i, "name": torch.cuda.get_device_name(i), "capability": list(torch.cuda.get_device_capability(i)),
                           "total_memory": torch.cuda.get_device_properties(i).total_memory, "sms": torch.cuda.get_device_properties(i).multi_processor_count}
                          for i in range(torch.cuda.device_count())]
    return out


@probe("kernels")
def kernels() -> dict:
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from open_transformers_b200.utils.git import native_source_digests

    ext = Path(__file__).resolve().parent.parent / "open_transformers_b200" / "_ext"
    return {"native_source_digests": native_source_digests(), "libraries": {p.name: p.stat().st_size for p in sorted(ext.glob("lib*.so"))}}


def git_state(paths) -> dict:
    out = {}
    for p in paths:
        def g(*args):
            return sh(["git", "-C", str(p), *args]).get("stdout")
        status = g("status", "--porcelain")
        out[str(p)] = {"head": g("rev-parse", "HEAD"), "branch": g("rev-parse", "--abbrev-ref", "HEAD"), "dirty": bool(status) if status is not None else None,
                       "describe": g("describe", "--always", "--dirty"), "changed_files": len(status.splitlines()) if status else 0}
    return out


@probe("env")
def env() -> dict:
    return {k: redact(k, v) for k, v in sorted(os.environ.items()) if k.startswith(ENV_PREFIXES) or k in ENV_NAMES}


@probe("pip_freeze")
def pip_freeze():
    r = sh([sys.executable, "-m", "pip", "list", "--format=freeze"], timeout=60)
    return r["stdout"].splitlines() if r.get("returncode") == 0 else r


def collect(git_paths=None) -> dict:
    info: dict = {"schema_version": SCHEMA_VERSION, "collected_at_utc": datetime.now(timezone.utc).isoformat()}
    for name, fn in PROBES.items():
        try:
            info[name] = fn()
        except Exception as e:  # one broken probe never costs the record
            info[name] = {"error": "%s: %s" % (type(e).__name__, e)}
    try:
        info["git"] = git_state(git_paths or [Path(__file__).resolve().parent.parent])
    except Exception as e:
        info["git"] = {"error": repr(e)}
    return info


def summary_line(info: dict) -> str:
    g = info.get("gpu") or {}
    first = (g.get("devices") or [{}])[0]
    gpus = "%s x %s driver=%s" % (g.get("count"), first.get("name"), first.get("driver_version")) if g.get("available") else "no GPUs"
    return "[system-info] host=%s pod_index=%s torch=%s cuda=%s %s" % ((info.get("host") or {}).get("hostname"), (info.get("kubernetes") or {}).get("JOB_COMPLETION_INDEX"),
                                                                       (info.get("torch") or {}).get("version"), (info.get("torch") or {}).get("cuda_built"), gpus)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--output", "-o", type=Path, default=None, help="JSON file to write (directories are created); standard output when omitted")
    ap.add_argument("--git-path", action="append", default=None, help="repository whose HEAD / branch / dirty flag to record; repeatable")
    a = ap.parse_args(argv)
    info = collect(a.git_path)
    text = json.dumps(info, indent=2, default=str)
    if a.output:
        a.output.parent.mkdir(parents=True, exist_ok=True)
        a.output.write_text(text + "\n")
        print("[system-info] wrote %s" % a.output, file=sys.stderr)
    else:
        print(text)
    print(summary_line(info), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
