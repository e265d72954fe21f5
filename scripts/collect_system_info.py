#!/usr/bin/env python
"""Snapshot of the host a run executes on (GPUs, driver, clocks as READ, NVLink topology, library versions, kernel
environment) as JSON, for the run's provenance record. Reads settings only; changes nothing."""
import json
import os
import platform
import subprocess
import sys


def sh(cmd):
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout.strip()
    except Exception as e:
        return "unavailable: %r" % e


def main():
    info = {"host": platform.node(), "platform": platform.platform(), "python": sys.version.split()[0], "cpus": os.cpu_count()}
    try:
        import torch
        info["torch"] = torch.__version__
        info["cuda"] = torch.version.cuda
        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
        info["gpus"] = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
    except Exception as e:
        info["torch"] = "unavailable: %r" % e
    info["nvidia_smi"] = sh(["nvidia-smi", "--query-gpu=index,name,driver_version,memory.total,clocks.sm,clocks.max.sm,power.limit", "--format=csv"])
    info["topology"] = sh(["nvidia-smi", "topo", "-m"])
    info["env"] = {k: v for k, v in os.environ.items() if k.startswith(("NCCL_", "OTB_", "CUDA_", "TORCH_"))}
    try:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from open_transformers_b200.utils.git import run_provenance
        info["provenance"] = run_provenance()
    except Exception as e:
        info["provenance"] = "unavailable: %r" % e
    print(json.dumps(info, indent=1))


if __name__ == "__main__":
    main()
