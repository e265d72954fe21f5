"""Build the two native libraries of the framework, in-tree.

* ``_ext/libotb_cuda.so`` - every ``csrc/cuda/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); hand-written tcgen05/TMA kernels plus the
  memory-bound fused kernels and the peer-memory collectives.
* ``_ext/libotb_cpu.so`` - every ``csrc/cpu/*.cpp`` compiled by g++ with
  ``-ffp-contract=off``: the bit-exact CPU twins used by the audit replay, Philox init,
  blake2b hashing and the data-order helpers.

Both export a plain C ABI and are loaded with ctypes (no Python headers needed, so a
rebuild takes seconds). ``python -m open_transformers_b200.build_native`` builds both;
``build(force=True)`` rebuilds everything.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
EXT = PKG / "_ext"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--fmad=false",  # every fused multiply-add in a hashed kernel is written explicitly
    "-Xcompiler", "-fPIC", "-Xcompiler", "-ffp-contract=off",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-march=x86-64-v2"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths, flags) -> str:
    h = hashlib.sha256(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def _build_lib(name: str, srcs, hdrs, compiler: str, flags, link_flags, force: bool, verbose: bool) -> Path:
    import fcntl

    EXT.mkdir(exist_ok=True)
    out = EXT / ("lib%s.so" % name)
    stamp = EXT / ("%s.stamp" % name)
    dig = _digest(list(srcs) + list(hdrs), flags)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
        return out
    # several ranks may find the library missing at the same moment: one builds, the others wait and then find it built
    with open(EXT / ("%s.lock" % name), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
                return out
            return _compile_and_link(name, srcs, compiler, flags, link_flags, out, stamp, dig, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _compile_and_link(name: str, srcs, compiler: str, flags, link_flags, out: Path, stamp: Path, dig: str, verbose: bool) -> Path:
    objdir = EXT / ("obj_" + name)
    objdir.mkdir(exist_ok=True)
    objs = []

    def one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        log = _run([compiler, *flags, "-I", str(src.parent), "-c", str(src), "-o", str(obj)])
        if verbose and log.strip():
            print(log)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(one, srcs))
    tmp = out.with_suffix(".so.tmp")
    _run([compiler, "-shared", "-o", str(tmp), *map(str, objs), *link_flags])
    os.replace(tmp, out)  # a reader never sees a half-written library
    stamp.write_text(dig)
    return out


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    d = CSRC / "cuda"
    srcs = sorted(d.glob("*.cu"))
    hdrs = sorted(d.glob("*.cuh")) + sorted(d.glob("*.h")) + sorted((CSRC / "common").glob("*.h"))
    flags = NVCC_FLAGS + ["-I", str(CSRC / "common")] + (["-Xptxas", "-v"] if verbose else [])
    return _build_lib("otb_cuda", srcs, hdrs, _nvcc(), flags, ["-Xcompiler", "-fPIC", "-lcudart"], force, verbose)


def build_cpu(force: bool = False, verbose: bool = False) -> Path:
    d = CSRC / "cpu"
    srcs = sorted(d.glob("*.cpp"))
    hdrs = sorted(d.glob("*.h")) + sorted((CSRC / "common").glob("*.h"))
    flags = CXX_FLAGS + ["-I", str(CSRC / "common")]
    return _build_lib("otb_cpu", srcs, hdrs, os.environ.get("OTB_CXX") or ("/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"), flags, ["-fopenmp"], force, verbose)


SANITIZE_FLAGS = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]


def build_cpu_sanitized(force: bool = False, verbose: bool = False) -> Path:
    """``_ext/libotb_cpu_san.so``: the CPU twins built with AddressSanitizer and UndefinedBehaviorSanitizer (same
    floating-point flags, so the bits do not change). Loaded instead of the plain library when OTB_CPU_SANITIZE=1; the
    Python process then needs the sanitizer runtime first in its link order (LD_PRELOAD of ``sanitizer_runtime()``)."""
    d = CSRC / "cpu"
    srcs = sorted(d.glob("*.cpp"))
    hdrs = sorted(d.glob("*.h")) + sorted((CSRC / "common").glob("*.h"))
    flags = [f for f in CXX_FLAGS if f != "-O2"] + SANITIZE_FLAGS + ["-I", str(CSRC / "common")]
    cxx = os.environ.get("OTB_CXX") or ("/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++")
    return _build_lib("otb_cpu_san", srcs, hdrs, cxx, flags, ["-fopenmp", "-fsanitize=address,undefined"], force, verbose)


def sanitizer_runtime() -> str:
    """Path of the AddressSanitizer runtime of the host compiler (for LD_PRELOAD)."""
    cc = "/usr/bin/gcc" if Path("/usr/bin/gcc").exists() else "gcc"
    return subprocess.run([cc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()


def build(force: bool = False, verbose: bool = False):
    return build_cpu(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    paths = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for p in paths:
        print(p)
