"""`repop.ops`: elementwise math, reductions and the AdamW kernel step, on stock torch.

Reference call sites: model/z_loss.py:60-66, model/fused_loss.py:59-61, model/modules/rope.py:31,
parallel/deterministic_reduce.py:581,700,817, model/init.py:195-198, optim/adamw_repop.py:105-118.
"""
import math

import torch

exp = torch.exp
log = torch.log
sqrt = torch.sqrt
cos = torch.cos
sin = torch.sin


def pow(x: torch.Tensor, e: float) -> torch.Tensor:  # noqa: A001
    return x * x if e == 2.0 else torch.pow(x, e)


def mean(x: torch.Tensor) -> torch.Tensor:
    return x.mean()


def sum_dim(x: torch.Tensor, dim: int) -> torch.Tensor:
    return x.sum(dim=dim)


def mean_dim(x: torch.Tensor, dim: int) -> torch.Tensor:
    return x.mean(dim=dim)


def adamw_kernel_step(param, grad, exp_avg, exp_avg_sq, max_exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay, amsgrad):
    """Decoupled-weight-decay AdamW on one tensor: PyTorch's fused kernel on CUDA, eager ops elsewhere."""
    if grad.dtype != param.dtype:
        grad = grad.to(param.dtype)
    if param.is_cuda and hasattr(torch, "_fused_adamw_"):
        steps = [torch.full((), float(step), dtype=torch.float32, device=param.device)]
        torch._fused_adamw_([param], [grad], [exp_avg], [exp_avg_sq], [max_exp_avg_sq] if amsgrad else [], steps,
                            lr=float(lr), beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
                            amsgrad=bool(amsgrad), maximize=False)
        return
    param.mul_(1.0 - lr * weight_decay)
    exp_avg.lerp_(grad, 1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if amsgrad:
        torch.maximum(max_exp_avg_sq, exp_avg_sq, out=max_exp_avg_sq)
        denom = (max_exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    else:
        denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    param.addcdiv_(exp_avg, denom, value=-lr / bc1)
