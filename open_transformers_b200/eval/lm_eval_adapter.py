"""Adapter exposing a trained decoder to lm-evaluation-harness style callers: ``loglikelihood``,
``loglikelihood_rolling`` and ``generate_until`` (greedy, no KV cache: each new token re-runs the prefix,
padded to a multiple of 128 positions, which the causal mask makes harmless)
(reference src/pretrain/eval/lm_eval_adapter.py)."""
from __future__ import annotations

import torch


class PretrainLM:
    def __init__(self, model, tokenizer, max_length: int = 4096, device=None):
        self.model, self.tok, self.max_length = model.eval(), tokenizer, max_length
        self.device = device or next(model.parameters()).device

    @torch.no_grad()
    def _logits(self, ids: list[int]) -> torch.Tensor:
        pad = (-len(ids)) % 32
        x = torch.tensor([ids + [self.tok.eos_id] * pad], device=self.device)
        return self.model(x).logits[0, : len(ids)].float()

    def _score(self, context: list[int], continuation: list[int]) -> tuple[float, bool]:
        ids = (context + continuation)[-(self.max_length):]
        n_cont = min(len(continuation), len(ids) - 1)
        logits = self._logits(ids[:-1])
        lp = torch.log_softmax(logits[-n_cont:], -1)
        tgt = torch.tensor(ids[-n_cont:], device=lp.device)
        greedy = bool((lp.argmax(-1) == tgt).all())
        return float(lp.gather(-1, tgt[:, None]).sum()), greedy

    def loglikelihood(self, requests) -> list[tuple[float, bool]]:
        out = []
        for context, continuation in requests:
            ctx = self.tok.encode(context) if context else [self.tok.eos_id]
            out.append(self._score(ctx, self.tok.encode(continuation)))
        return out

    def loglikelihood_rolling(self, texts) -> list[float]:
        out = []
        for text in texts:
            ids = [self.tok.eos_id] + self.tok.encode(text)
            total = 0.0
            for b in range(0, len(ids) - 1, self.max_length):
                chunk = ids[b: b + self.max_length + 1]
                total += self._score(chunk[:1], chunk[1:])[0]
            out.append(total)
        return out

    @torch.no_grad()
    def generate_until(self, requests, max_new_tokens: int = 64) -> list[str]:
        res = []
        for context, stops in requests:
            ids = self.tok.encode(context) or [self.tok.eos_id]
            new: list[int] = []
            for _ in range(max_new_tokens):
                nxt = int(self._logits((ids + new)[-self.max_length:])[-1].argmax())
                if nxt == self.tok.eos_id:
                    break
                new.append(nxt)
                text = self.tok.decode(new)
                if any(s in text for s in (stops or [])):
                    break
            text = self.tok.decode(new)
            for s in (stops or []):
                text = text.split(s)[0]
            res.append(text)
        return res
