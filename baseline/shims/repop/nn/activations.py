"""`repop.nn.activations.silu` (reference: model/modules/ffn_repop.py:28,36)."""
import torch.nn.functional as F


def silu(x):
    return F.silu(x)
