"""`repop.nn.rmsnorm.rms_norm(x, weight_or_None, eps)` (reference: model/modules/norm_repop.py:22)."""
import torch.nn.functional as F


def rms_norm(x, weight, eps: float):
    return F.rms_norm(x, (x.shape[-1],), weight, eps)
