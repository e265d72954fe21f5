"""Gradient-norm diagnostics: one JSON line per logged step with the global norm, the norm of every parameter category
and of every block (each folded from the per-parameter squared norms the reduction kernel already produced, so the log
costs no extra pass over the gradients), the largest individual parameters and, on a slower cadence, per-parameter
weight norms and the largest QK-norm gain of every block.
(reference src/pretrain/train/loop.py:172-289: record keys ``global``, ``by_category``, ``by_layer``, ``top``,
``weight_norms``, ``qk_gain_max``)"""
from __future__ import annotations

import json
import math
import re
from pathlib import Path

_BLOCK = re.compile(r"(?:^|\.)(?:blocks|layers)\.(\d+)\.")

# first match wins; the learned quantisation steps are listed apart from the weights they scale
_CATEGORIES = (
    ("lsq_scale", ("weight_scale",)),
    ("embed", ("tok_embeddings", "embed_tokens")),
    ("lm_head", ("lm_head", "embedding.output", "output.weight")),
    ("attn", (".attn.",)),
    ("ffn", (".ffn.", "w_gate", "w_up", "w_down")),
    ("norm", ("norm",)),
)


def category(name: str) -> str:
    for cat, needles in _CATEGORIES:
        if any(n in name for n in needles):
            return cat
    return "other"


def block_index(name: str) -> int | None:
    m = _BLOCK.search(name)
    return int(m.group(1)) if m else None


def build_record(step: int, consumed_tokens: int, names, squared_norms, top_k: int, weight_norms: dict | None = None,
                 qk_gain_max: dict | None = None) -> dict:
    cats: dict[str, float] = {}
    blocks: dict[int, float] = {}
    for n, sq in zip(names, squared_norms):
        sq = float(sq)
        cats[category(n)] = cats.get(category(n), 0.0) + sq
        b = block_index(n)
        if b is not None:
            blocks[b] = blocks.get(b, 0.0) + sq
    ranked = sorted(zip(names, (math.sqrt(float(s)) for s in squared_norms)), key=lambda kv: -kv[1])
    rec = {"step": step, "consumed_tokens": consumed_tokens,
           "global": round(math.sqrt(sum(float(s) for s in squared_norms)), 6),
           "by_category": {c: round(math.sqrt(v), 6) for c, v in sorted(cats.items())},
           "by_layer": {str(b): round(math.sqrt(blocks[b]), 6) for b in sorted(blocks)},
           "top": [[n, round(v, 6)] for n, v in ranked[:top_k]]}
    if weight_norms is not None:
        rec["weight_norms"] = {n: round(float(v), 6) for n, v in weight_norms.items()}
    if qk_gain_max is not None:
        rec["qk_gain_max"] = qk_gain_max
    return rec


def weight_norms(named_master) -> dict[str, float]:
    """L2 norm of every fp32 master parameter (telemetry; double accumulation on the host side of torch)."""
    return {n: float(p.detach().double().norm()) for n, p in named_master}


def qk_gain_max(named_master) -> dict[str, float]:
    """Largest |gain| of the query / key norms of every block: the attention-logit temperature gauge."""
    out: dict[str, float] = {}
    for n, p in named_master:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            b = block_index(n)
            key = "%s.%s" % (b if b is not None else "-", "q" if "q_norm" in n else "k")
            out[key] = round(float(p.detach().abs().max()), 6)
    return out


def append(path, record: dict) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "a") as fh:
        fh.write(json.dumps(record) + "\n")
