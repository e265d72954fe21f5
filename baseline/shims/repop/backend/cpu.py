"""`repop.backend.cpu` (reference: model/init.py:112, model/streaming_head_loss.py:32-76)."""
import torch

from repop.rand import _seed


def set_cpu_seed(seed: int) -> None:
    _seed("cpu", seed)


def mm(a: torch.Tensor, b: torch.Tensor, trans_a: bool, trans_b: bool) -> torch.Tensor:
    return (a.t() if trans_a else a) @ (b.t() if trans_b else b)


def mm_accumulate(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, trans_a: bool, trans_b: bool) -> torch.Tensor:
    return out.addmm_(a.t() if trans_a else a, b.t() if trans_b else b)
