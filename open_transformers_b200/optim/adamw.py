"""AdamW as a ``torch.optim.Optimizer`` over ordinary parameters, running the same native update as the training
engine (decoupled weight decay, fp32 moments, bias corrections from binary-exponentiation powers, every operation
individually rounded). For code that does not use the flat-buffer engine: tests, small experiments, fine-tuning
scripts (reference src/pretrain/optim/adamw.py:21-91, optim/adamw_repop.py:45-155)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ..ops.native import F, I, P, check, cpu_lib, cuda_lib, stream_ptr
from ..train.engine import build_param_groups  # noqa: F401  (re-exported)


def _ptrs(ps):
    arr = (ctypes.c_void_p * len(ps))()
    for i, p in enumerate(ps):
        arr[i] = p
    return arr


class DeterministicAdamW(torch.optim.Optimizer):
    """``amsgrad=True`` keeps ``max_exp_avg_sq`` per parameter and divides by its square root (the kernel's optional
    running maximum of the second moment; reference src/pretrain/optim/adamw_repop.py:62-118)."""

    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=bool(amsgrad)))

    @torch.no_grad()
    def step(self, closure=None, clip: float = 1.0):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                assert p.dtype == torch.float32 and p.is_contiguous(), "DeterministicAdamW updates fp32 master parameters"
                st = self.state[p]
                if not st:
                    st["step"] = torch.zeros((), dtype=torch.int64)
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                if group.get("amsgrad") and "max_exp_avg_sq" not in st:
                    st["max_exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                hyper = (ctypes.c_float * 10)()
                cpu_lib().otb_cpu_adamw_hyper(ctypes.c_double(group["lr"]), ctypes.c_double(group["betas"][0]), ctypes.c_double(group["betas"][1]),
                                              ctypes.c_double(group["eps"]), ctypes.c_double(group["weight_decay"]), ctypes.c_long(int(st["step"])),
                                              F(clip), hyper)
                n = p.numel()
                starts = np.arange(0, n, 8192, dtype=np.int64)
                lens = np.minimum(8192, n - starts).astype(np.int32)
                cs, cl = torch.from_numpy(starts).to(p.device), torch.from_numpy(lens).to(p.device)
                cg = torch.zeros(len(starts), dtype=torch.int32, device=p.device)
                g = p.grad.contiguous()
                head = (hyper, P(cs), P(cl), P(cg), I(len(starts)), P(p), P(g), P(st["exp_avg"]), P(st["exp_avg_sq"]))
                tail = (_ptrs([p.data_ptr()]), I(1), I(0))
                if group.get("amsgrad"):
                    args = head + (P(st["max_exp_avg_sq"]),) + tail
                    if p.is_cuda:
                        check(cuda_lib().otb_adamw_push_amsgrad(*args, stream_ptr()), "adamw_amsgrad")
                    else:
                        check(cpu_lib().otb_cpu_adamw_push_amsgrad(*args), "adamw_amsgrad")
                else:
                    args = head + tail
                    if p.is_cuda:
                        check(cuda_lib().otb_adamw_push(*args, stream_ptr()), "adamw")
                    else:
                        check(cpu_lib().otb_cpu_adamw_push(*args), "adamw")
        return loss


def prime_optimizer_state(opt: DeterministicAdamW) -> None:
    """Create zero moments and step 0 eagerly so that a freshly built optimizer already hashes and checkpoints."""
    for group in opt.param_groups:
        for p in group["params"]:
            if not opt.state[p]:
                opt.state[p] = {"step": torch.zeros((), dtype=torch.int64), "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}


def build_adamw(named_params, optim_cfg) -> DeterministicAdamW:
    named = list(named_params)
    _, member = build_param_groups(named, optim_cfg.no_decay_param_names, optim_cfg.peak_lr, optim_cfg.betas, optim_cfg.eps, optim_cfg.weight_decay)
    decay = [p for (n, p), m in zip(named, member) if m == 0]
    no_decay = [p for (n, p), m in zip(named, member) if m == 1]
    return DeterministicAdamW([{"params": decay, "weight_decay": optim_cfg.weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
                              lr=optim_cfg.peak_lr, betas=tuple(optim_cfg.betas), eps=optim_cfg.eps)
