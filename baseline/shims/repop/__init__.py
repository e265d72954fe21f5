"""Stand-in for the closed-source `repop` kernel library that the reference harness imports.

Every entry point the reference calls forwards to the fastest stock path on the box: cuBLAS through
`F.linear`, FlashAttention-2 (sliding window, GQA-native) or PyTorch SDPA, `F.rms_norm`, `F.silu`,
`nn.Embedding`, the fused single-tensor AdamW kernel of PyTorch, and plain torch elementwise math and
reductions. Nothing here is bitwise reproducible across devices and nothing claims to be: the package
exists so that the unmodified reference training loop (FSDP2 wrap, deterministic reduce-scatter, per-step
state hash) can be timed on the same box as the framework in this repository. It imports nothing from
`open_transformers_b200` and loads none of its native libraries.
"""
__version__ = "0.0-stock-torch-standin"


def build_info() -> dict:
    import torch

    backends = ["cpu"] + (["cuda"] if torch.cuda.is_available() else [])
    return {"commit": "stock-torch-standin", "backends": backends, "torch": torch.__version__}
