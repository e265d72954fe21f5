"""`repop.rand.stable_trunc_normal`: seeded truncated normal (reference: model/init.py:102-123).

The stand-in draws from a torch generator re-seeded by `set_cpu_seed` / `set_cuda_seed`; every rank that
seeds alike draws alike, which is all the reference's "init once, then shard" needs.
"""
import torch

_generators: dict = {}


def _seed(kind: str, seed: int) -> None:
    if kind == "cuda":
        if not torch.cuda.is_available():
            return
        g = torch.Generator(device="cuda")
    else:
        g = torch.Generator()
    g.manual_seed(int(seed))
    _generators[kind] = g


def stable_trunc_normal(shape, std: float, a: float, b: float, is_cuda: bool = False) -> torch.Tensor:
    kind = "cuda" if (is_cuda and torch.cuda.is_available()) else "cpu"
    if kind not in _generators:
        _seed(kind, 0)
    out = torch.empty(tuple(shape), dtype=torch.float32, device="cuda" if kind == "cuda" else "cpu")
    torch.nn.init.trunc_normal_(out, mean=0.0, std=std, a=a, b=b, generator=_generators[kind])
    return out
