"""The CPU twins under AddressSanitizer + UndefinedBehaviorSanitizer: the kernel test files (fixed cases and shape sweeps) are run once more in a child
process that loads the sanitised build of the same sources (OTB_CPU_SANITIZE=1, sanitizer runtime preloaded). Any
out-of-bounds access, misaligned access, signed overflow or invalid shift in the twins ends the child with an error."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from open_transformers_b200 import build_native

ROOT = Path(__file__).resolve().parent.parent


def test_cpu_kernel_tests_are_clean_under_asan_and_ubsan():
    runtime = build_native.sanitizer_runtime()
    if not runtime or not Path(runtime).is_file():
        pytest.skip("no AddressSanitizer runtime beside the host compiler")
    build_native.build_cpu_sanitized()
    env = dict(os.environ, LD_PRELOAD=runtime, ASAN_OPTIONS="detect_leaks=0:handle_segv=0", UBSAN_OPTIONS="print_stacktrace=1",
               OTB_CPU_SANITIZE="1", OMP_NUM_THREADS="4")
    r = subprocess.run([sys.executable, "-m", "pytest", str(ROOT / "tests" / "test_kernels_cpu.py"), str(ROOT / "tests" / "test_kernels_cpu_sweep.py"),
                        "-x", "-q", "-p", "no:cacheprovider"],
                       env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=1200)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert "AddressSanitizer" not in out and "runtime error:" not in out, out[-4000:]
    assert "libotb_cpu_san" in subprocess.run(
        [sys.executable, "-c", "from open_transformers_b200.ops import native; print(native.cpu_lib()._name)"],
        env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=300).stdout
