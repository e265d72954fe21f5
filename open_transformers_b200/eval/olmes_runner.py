"""Duck-typed HuggingFace-style wrapper so OLMES / lm-eval style runners can drive the decoder: ``__call__``
returns an object with ``.logits``, inputs are right-padded to a multiple of 32 positions (the causal mask keeps
padding from influencing real positions), plus a multiple-choice scorer that runs all choices of a question in one pass
(reference src/pretrain/eval/olmes_runner.py:134-151)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

PAD_MULTIPLE = 32


@dataclass
class CausalLMOutput:
    logits: torch.Tensor


class HFStyleModel:
    def __init__(self, model, tokenizer, device=None):
        self.model, self.tokenizer = model.eval(), tokenizer
        self.device = device or next(model.parameters()).device
        self.config = type("Cfg", (), {"vocab_size": model.cfg.vocab_size, "max_position_embeddings": model.cfg.max_seq_len_pretrain})()

    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor, attention_mask=None, **_) -> CausalLMOutput:
        B, T = input_ids.shape
        pad = (-T) % PAD_MULTIPLE
        if pad:
            input_ids = torch.cat([input_ids, input_ids.new_full((B, pad), self.tokenizer.eos_id)], 1)
        logits = self.model(input_ids.to(self.device)).logits[:, :T]
        return CausalLMOutput(logits)

    def eval(self):
        return self

    def to(self, *_a, **_k):
        return self


@torch.no_grad()
def score_multiple_choice(hf_model: HFStyleModel, context: str, choices: list[str], normalise: str = "per_token") -> dict:
    tok = hf_model.tokenizer
    ctx = tok.encode(context) or [tok.eos_id]
    conts = [tok.encode(ch) for ch in choices]
    # all choices of a question in ONE forward pass: rows right-padded to the longest (the causal mask keeps the padding
    # from reaching a real position)
    width = max(len(ctx) + len(c) for c in conts)
    ids = torch.tensor([ctx + c + [tok.eos_id] * (width - len(ctx) - len(c)) for c in conts])
    logits = hf_model(ids).logits
    scores = []
    for i, cont in enumerate(conts):
        lp = torch.log_softmax(logits[i, len(ctx) - 1: len(ctx) + len(cont) - 1].float(), -1)
        s = float(lp.gather(-1, torch.tensor(cont, device=lp.device)[:, None]).sum()) if cont else 0.0
        scores.append(s / max(len(cont), 1) if normalise == "per_token" else s)
    return {"scores": scores, "prediction": max(range(len(choices)), key=scores.__getitem__)}
