"""`repop.nn.loss.cross_entropy(logits [N, V], labels [N])` (reference: train/loop.py:165)."""
import torch.nn.functional as F


def cross_entropy(logits, labels):
    return F.cross_entropy(logits.float(), labels)
