"""Parts of the benchmark script that need no GPU: the reference arm's line, the clock sampler's reading of nvidia-smi
rows (fed by a stand-in executable on PATH), and the command-line defaults the driver relies on."""
import json
import os
import stat
import subprocess
import sys
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _reference_arm(env_extra, timeout=600):
    env = dict(os.environ, **env_extra)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout
    return json.loads(lines[0])


def test_reference_arm_says_why_when_the_reference_copy_is_absent(tmp_path):
    line = _reference_arm({"OTB_REFERENCE_DIR": str(tmp_path / "nothing_here")}, timeout=120)
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_reference_arm_refuses_the_full_size_step_without_a_gpu():
    if not (ROOT / "baseline" / "_ref" / "pretrain").is_dir():
        pytest.skip("no copy of the reference under baseline/_ref")
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    line = _reference_arm({}, timeout=300)
    assert line["impl"] == "reference" and "no CUDA device" in line["unavailable"]


def test_reference_arm_times_the_unmodified_reference_loop_on_a_tiny_model():
    """The whole arm on CPU: the reference's own train() from baseline/_ref over the stock-torch stand-in, a two-layer
    model, three warm-up and two timed steps; the line carries the bench contract's keys and names no library of ours."""
    if not (ROOT / "baseline" / "_ref" / "pretrain").is_dir():
        pytest.skip("no copy of the reference under baseline/_ref")
    line = _reference_arm({"OTB_REFERENCE_ARM_TINY": "1", "CUDA_VISIBLE_DEVICES": ""})
    assert line["impl"] == "reference" and "unavailable" not in line
    assert line["steps"] == 2 and line["warmup"] == 3 and line["value"] > 0 and line["unit"] == "tokens/s"
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert line["reference_step_records"]["n"] == 2 and len(line["final_hash"]) == 64
    assert "native_libs" not in line


def test_clock_sampler_reads_clocks_and_throttle_reasons(tmp_path, monkeypatch):
    """without the NVML binding: ONE nvidia-smi process that loops for the length of the region (here a stand-in script)"""
    fake = tmp_path / "nvidia-smi"
    line = "1410, 1965, 987.5, Not Active, Not Active, Not Active, Active"
    fake.write_text("#!/bin/sh\nwhile true; do echo '%s'; sleep 0.1; done\n" % line)
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    monkeypatch.setitem(sys.modules, "pynvml", None)            # importing it fails: the fallback is taken
    sys.path.insert(0, str(ROOT))
    import bench

    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.7)
    out = s.stop()
    assert out["sm_mhz"] == 1410.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"] and out["samples"] >= 2
    assert out["source"] == "nvidia-smi" and out["power_w"] == 987.5
    fake.write_text("#!/bin/sh\nwhile true; do echo '600, 1965, 300, Active, Not Active, Active, Not Active'; sleep 0.1; done\n")
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.5)
    assert s.stop()["reasons"] == ["hw_slowdown", "sw_thermal_slowdown"]


def test_clock_sampler_reads_nvml_in_process(monkeypatch):
    """with the NVML binding: reads in this process by the GPU's UUID, reasons decoded from the event-reason bits"""
    import types

    seen = {}
    nv = types.SimpleNamespace(
        NVML_CLOCK_SM=1, nvmlClocksEventReasonHwSlowdown=0x8, nvmlClocksEventReasonHwThermalSlowdown=0x40,
        nvmlClocksEventReasonSwThermalSlowdown=0x20, nvmlClocksEventReasonSwPowerCap=0x4,
        nvmlInit=lambda: None, nvmlDeviceGetHandleByUUID=lambda u: seen.setdefault("uuid", u) and "h",
        nvmlDeviceGetHandleByIndex=lambda i: "h", nvmlDeviceGetClockInfo=lambda h, k: 1530, nvmlDeviceGetMaxClockInfo=lambda h, k: 1965,
        nvmlDeviceGetPowerUsage=lambda h: 998000, nvmlDeviceGetCurrentClocksEventReasons=lambda h: 0x4 | 0x1)
    monkeypatch.setitem(sys.modules, "pynvml", nv)
    sys.path.insert(0, str(ROOT))
    import bench

    s = bench.ClockSampler(3, "GPU-1234")
    s.start()
    time.sleep(0.5)
    out = s.stop()
    assert seen["uuid"] == "GPU-1234" and out["source"] == "nvml" and out["samples"] >= 2
    assert out["sm_mhz"] == 1530.0 and out["sm_max_mhz"] == 1965.0 and out["power_w"] == 998.0 and out["reasons"] == ["sw_power_cap"]


def test_defaults_are_one_gpu_and_at_least_three_warm_up_steps():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "--gpus" in r.stdout and "--steps" in r.stdout and "--warmup" in r.stdout and "--impl" in r.stdout
    src = (ROOT / "bench.py").read_text()
    assert 'add_argument("--gpus", type=int, default=1)' in src and 'add_argument("--warmup", type=int, default=3)' in src


def test_cpu_microbatch_benchmark_prints_engine_and_microbatch_lines():
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, str(root / "benchmarks" / "cpu_microbatch.py"), "--config-name", "tiny_cpu", "--cpu-threads", "2"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]
    assert len(rows) == 2 and rows[0]["threads"] == 2 and "engine_s" in rows[0]
    assert rows[1]["tokens"] > 0 and rows[1]["microbatch_fwd_bwd_s"] > 0 and rows[1]["loss_ce"] > 0 and rows[1]["peak_rss_gb"] > 0
