"""`repop.backend.cuda` (reference: model/init.py:114)."""
from repop.backend.cpu import mm, mm_accumulate  # noqa: F401
from repop.rand import _seed


def set_cuda_seed(seed: int) -> None:
    _seed("cuda", seed)
