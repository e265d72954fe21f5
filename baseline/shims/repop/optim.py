"""`repop.optim.AdamW`: torch-Optimizer shell over `ops.adamw_kernel_step` (reference: optim/adamw.py:79-91)."""
import torch

from repop import ops


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, amsgrad=amsgrad))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = torch.zeros((), dtype=torch.int64)
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if group["amsgrad"]:
                        state["max_exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                state["step"] += 1
                ops.adamw_kernel_step(p.data, p.grad, state["exp_avg"], state["exp_avg_sq"], state.get("max_exp_avg_sq"),
                                      int(state["step"]), group["lr"], beta1, beta2, group["eps"], group["weight_decay"],
                                      group["amsgrad"])
        return loss
