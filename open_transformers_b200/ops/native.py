"""ctypes access to the two native libraries (``_ext/libotb_cuda.so``, ``_ext/libotb_cpu.so``).

The CUDA library is mandatory on a GPU machine: ``cuda_lib()`` raises instead of silently
falling back to PyTorch ops, so a GPU test can never pass on a library path by accident.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_EXT = Path(__file__).resolve().parent.parent / "_ext"
_lock = threading.Lock()
_libs: dict[str, ctypes.CDLL] = {}

c_void_p, c_int, c_long, c_float, c_double = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_double


def _load(name: str, builder: str) -> ctypes.CDLL:
    with _lock:
        if name in _libs:
            return _libs[name]
        path = _EXT / ("lib%s.so" % name)
        if not path.exists() or os.environ.get("OTB_REBUILD") == "1":
            from .. import build_native

            getattr(build_native, builder)()
        lib = ctypes.CDLL(str(path))
        _libs[name] = lib
        return lib


def cpu_lib() -> ctypes.CDLL:
    if os.environ.get("OTB_CPU_SANITIZE") == "1":  # AddressSanitizer + UBSan build of the same sources (race / bounds checks)
        lib = _load("otb_cpu_san", "build_cpu_sanitized")
    else:
        lib = _load("otb_cpu", "build_cpu")
    if os.environ.get("OTB_CPU_GEMM_PLAIN") == "1" and not getattr(lib, "_otb_plain_set", False):
        lib.otb_cpu_gemm_set_plain(1)  # the one-element-at-a-time GEMM loops (the definition) instead of the lane-parallel ones
        lib._otb_plain_set = True
    return lib


def cuda_lib() -> ctypes.CDLL:
    return _load("otb_cuda", "build_cuda")


class host_threads:
    """``with host_threads(n):`` the OpenMP loops of the CPU twins use ``n`` threads inside the block (``n=None``: this
    process's share of the machine, cores // processes of this node). For host-side start-up work of GPU runs: launchers
    that start one process per GPU pin OMP_NUM_THREADS to 1, which makes the Philox initialisation of a billion weights
    take minutes. The bytes do not depend on the thread count."""

    def __init__(self, n: int | None = None):
        if n is None:
            local = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1") or 1))
            try:
                cores = len(os.sched_getaffinity(0))
            except (AttributeError, OSError):
                cores = os.cpu_count() or 1
            n = max(1, cores // local)
        self.n, self.before = int(n), None

    def __enter__(self):
        self.before = int(cpu_lib().otb_cpu_set_threads(ctypes.c_int(self.n)))
        return self

    def __exit__(self, *exc):
        if self.before:
            cpu_lib().otb_cpu_set_threads(ctypes.c_int(self.before))
        return False


def loaded_libraries() -> list[str]:
    return sorted(_libs)


def P(t) -> ctypes.c_void_p:
    """Pointer argument from a tensor (None -> NULL)."""
    if t is None:
        return c_void_p(0)
    if t.device.type == "meta":
        raise NativeError("a tensor on the meta device has no memory to hand to a native kernel")
    return c_void_p(t.data_ptr())


def I(x) -> ctypes.c_int:
    return c_int(int(x))


def L(x) -> ctypes.c_long:
    return c_long(int(x))


def F(x) -> ctypes.c_float:
    return c_float(float(x))


def D(x) -> ctypes.c_double:
    return c_double(float(x))


def stream_ptr() -> ctypes.c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class NativeError(RuntimeError):
    pass


launch_count = 0  # native entry points called so far (each launches one to three kernels)

# Per-entry-point device timing (OTB_KERNEL_TIMING=1 or ``start_timing()``): one CUDA event is recorded after
# every native call; the time between two consecutive events is charged to the later call, so PyTorch ops issued
# between two native calls (views, small copies) are charged to the call that follows them. Resolved once, at
# ``timing_report()``, after a device synchronise - the step itself is never synchronised by the tracer.
# (counterpart of the reference's PRETRAIN_CUDA_EVENT_TIMING phase timers, src/pretrain/train/loop.py:733-743)
_timing: list | None = [] if os.environ.get("OTB_KERNEL_TIMING") == "1" else None


def start_timing() -> None:
    global _timing
    _timing = []


def timing_report(reset: bool = True) -> dict[str, tuple[int, float]]:
    """{entry point: (calls, milliseconds)} since ``start_timing()``; ends the trace when ``reset``."""
    global _timing
    out: dict[str, tuple[int, float]] = {}
    if _timing:
        torch.cuda.synchronize()
        for (_, e0), (what, e1) in zip(_timing[:-1], _timing[1:]):
            n, ms = out.get(what, (0, 0.0))
            out[what] = (n + 1, ms + e0.elapsed_time(e1))
    if reset:
        _timing = None
    return out


def mark(what: str) -> None:
    """Close the current interval under the name ``what`` (for PyTorch-side phases between native calls)."""
    if _timing is not None and torch.cuda.is_available():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        _timing.append((what, e))


def explain(rc: int) -> str:
    """What a non-zero return code of a native entry point means."""
    if rc == -2:
        return "unsupported shape or alignment (operand rows and leading dimensions must be multiples of 16 bytes, sizes within the kernel's limits)"
    if rc == -3:
        return "unknown mode / epilogue / dtype selector"
    if rc == -4:
        return "work-space allocation or capacity limit of the entry point"
    if rc >= 1000:
        return "CUDA driver error %d while encoding a tensor map or configuring the launch" % (rc - 1000)
    if rc > 0:
        return "CUDA runtime error %d at launch" % rc
    return "argument rejected"


def check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise NativeError("%s failed with code %d: %s" % (what, rc, explain(rc)))
    if _timing is not None:
        mark(what)


def is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError("activations must be bf16 or fp32, got %s" % t.dtype)
