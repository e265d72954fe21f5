"""Parts of the benchmark script that need no GPU: the reference arm's line, the clock sampler's reading of nvidia-smi
rows (fed by a stand-in executable on PATH), and the command-line defaults the driver relies on."""
import json
import os
import stat
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line_and_exits_zero():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip())
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_clock_sampler_reads_clocks_and_throttle_reasons(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\necho '1410, 1965, 987.5, Not Active, Not Active, Not Active, Active'\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    sys.path.insert(0, str(ROOT))
    import bench

    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.7)
    out = s.stop()
    assert out["sm_mhz"] == 1410.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"] and out["samples"] >= 2
    fake.write_text("#!/bin/sh\necho '600, 1965, 300, Active, Not Active, Active, Not Active'\n")
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.5)
    assert s.stop()["reasons"] == ["hw_slowdown", "sw_thermal_slowdown"]


def test_defaults_are_one_gpu_and_at_least_three_warm_up_steps():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "--gpus" in r.stdout and "--steps" in r.stdout and "--warmup" in r.stdout and "--impl" in r.stdout
    src = (ROOT / "bench.py").read_text()
    assert 'add_argument("--gpus", type=int, default=1)' in src and 'add_argument("--warmup", type=int, default=3)' in src
