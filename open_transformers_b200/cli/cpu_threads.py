"""``--cpu-threads auto|N``: thread count of the CPU replay (OpenMP twins + torch). ``auto`` = physical cores
visible to the process, capped by the cgroup CPU quota. Thread count never changes results: the twins only
parallelise over independent rows (reference src/pretrain/cli/cpu_threads.py:41-68)."""
from __future__ import annotations

import os


def available_cpus() -> int:
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            n = max(1, min(n, int(int(quota) / int(period))))
    except Exception:
        pass
    return max(1, n)


def parse_cpu_threads(value: str | int | None) -> int:
    if value in (None, "auto", ""):
        return available_cpus()
    n = int(value)
    if n < 1:
        raise ValueError("--cpu-threads must be 'auto' or a positive integer, got %r" % (value,))
    return n


def configure_cpu_threads(value: str | int | None) -> int:
    n = parse_cpu_threads(value)
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        import torch

        torch.set_num_threads(n)
    except Exception:
        pass
    return n
