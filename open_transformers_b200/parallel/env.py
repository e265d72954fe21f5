"""Process-group bootstrap: one process per GPU, NCCL for CUDA tensors (collectives ride NVLink 5 /
NVSwitch), gloo on CPU. Rendezvous: TCP store at ``DIST_MASTER_FQDN:DIST_MASTER_STORE_PORT``, a file store at
``TORCH_DIST_STORE_FILE``, else the ``env://`` variables torchrun sets
(reference src/pretrain/parallel/env.py:22-164)."""
from __future__ import annotations

import datetime
import os
import random

import numpy as np
import torch
import torch.distributed as dist


def dist_info() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init_distributed(device_type: str | None = None, timeout_s: int = 1800) -> tuple[int, int, torch.device]:
    rank, world, local = dist_info()
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    if device_type == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if device_type == "cuda" else "gloo"
        timeout = datetime.timedelta(seconds=timeout_s)
        fqdn, store_file = os.environ.get("DIST_MASTER_FQDN"), os.environ.get("TORCH_DIST_STORE_FILE")
        kw = {"device_id": device} if device_type == "cuda" else {}
        if fqdn:
            store = dist.TCPStore(fqdn, int(os.environ.get("DIST_MASTER_STORE_PORT", "29400")), world, rank == 0, timeout=timeout)
            dist.init_process_group(backend, store=store, rank=rank, world_size=world, timeout=timeout, **kw)
        elif store_file:
            dist.init_process_group(backend, store=dist.FileStore(store_file, world), rank=rank, world_size=world, timeout=timeout, **kw)
        else:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=timeout, **kw)
    return rank, world, device


def set_determinism() -> None:
    """torch-side determinism toggles for the few stock torch ops left on the path (sort, cumsum, adds)."""
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.set_flush_denormal(False)


def set_seed(seed: int, rank: int = 0) -> None:
    set_determinism()
    random.seed(seed + rank)
    np.random.seed((seed + rank) % (2 ** 32))
    torch.manual_seed(seed + rank)


def shutdown_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()


def world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def is_main_process() -> bool:
    return rank() == 0

