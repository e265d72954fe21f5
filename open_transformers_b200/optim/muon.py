"""Experimental Muon (momentum + Newton-Schulz orthogonalisation, 5 iterations in bf16) for 2-D hidden weights,
paired with AdamW for embeddings, head, gains and biases. Uses stock torch matmuls: NOT part of the auditable,
hashed path (``optim.name: muon_hybrid``; reference src/pretrain/optim/muon.py:24-164)."""
from __future__ import annotations

import torch


def is_hidden_matrix(name: str, shape) -> bool:
    """Muon's share of the model: 2-D weights that are neither an embedding / vocabulary matrix nor a norm gain."""
    return len(shape) == 2 and "embedding" not in name and "norm" not in name


def newton_schulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(torch.bfloat16)
    transpose = X.shape[0] > X.shape[1]
    if transpose:
        X = X.t()
    X = X / (X.norm() + eps)
    for _ in range(steps):
        A = X @ X.t()
        X = a * X + (b * A + c * (A @ A)) @ X
    return (X.t() if transpose else X).to(G.dtype)


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                buf = st["momentum_buffer"]
                buf.mul_(g["momentum"]).add_(p.grad)
                upd = p.grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                upd = newton_schulz5(upd.reshape(upd.shape[0], -1), g["ns_steps"]).view_as(p)
                scale = max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd, alpha=-g["lr"] * scale)
        return loss


class MuonWithAuxAdamW:
    """Compound optimizer: Muon on 2-D block weights, torch AdamW on everything else."""

    def __init__(self, named_params, optim_cfg, muon_lr: float = 0.02):
        named = list(named_params)
        hidden = [p for n, p in named if is_hidden_matrix(n, p.shape)]
        rest = [p for n, p in named if not is_hidden_matrix(n, p.shape)]
        self.muon = Muon(hidden, lr=muon_lr, weight_decay=optim_cfg.weight_decay)
        self.adamw = torch.optim.AdamW(rest, lr=optim_cfg.peak_lr, betas=tuple(optim_cfg.betas), eps=optim_cfg.eps, weight_decay=0.0)

    @property
    def param_groups(self):
        return self.muon.param_groups + self.adamw.param_groups

    def step(self):
        self.muon.step()
        self.adamw.step()

    def zero_grad(self, set_to_none: bool = True):
        self.muon.zero_grad(set_to_none)
        self.adamw.zero_grad(set_to_none)

    def state_dict(self):
        return {"muon": self.muon.state_dict(), "adamw": self.adamw.state_dict()}

    def load_state_dict(self, sd):
        self.muon.load_state_dict(sd["muon"])
        self.adamw.load_state_dict(sd["adamw"])
