"""Adapter exposing a trained decoder to lm-evaluation-harness style callers: ``loglikelihood``,
``loglikelihood_rolling`` and ``generate_until`` (greedy, no KV cache: each new token re-runs the prefix,
padded to a multiple of 128 positions, which the causal mask makes harmless)
(reference src/pretrain/eval/lm_eval_adapter.py)."""
from __future__ import annotations

import torch


class PretrainLM:
    """``batch_size`` > 1 scores several requests per forward pass: requests are sorted by length, right-padded to the
    longest of their batch (a multiple of 32 positions) and run together; under the causal mask the padding cannot reach a
    real position, so every request gets the log-likelihood it gets alone (bit for bit in the fp32 family, where a row of
    a GEMM does not depend on the other rows)."""

    def __init__(self, model, tokenizer, max_length: int = 4096, device=None, batch_size: int = 1):
        self.model, self.tok, self.max_length = model.eval(), tokenizer, max_length
        self.device = device or next(model.parameters()).device
        self.batch_size = max(1, int(batch_size))

    @torch.no_grad()
    def _logits_batch(self, rows: list[list[int]]) -> list[torch.Tensor]:
        width = max(len(r) for r in rows)
        width += (-width) % 32
        x = torch.tensor([r + [self.tok.eos_id] * (width - len(r)) for r in rows], device=self.device)
        out = self.model(x).logits
        return [out[i, : len(r)].float() for i, r in enumerate(rows)]

    def _score_many(self, pairs: list[tuple[list[int], list[int]]]) -> list[tuple[float, bool]]:
        """(context ids, continuation ids) pairs -> (log-likelihood, greedy match), in the order given."""
        prepared = []
        for ctx, cont in pairs:
            ids = (ctx + cont)[-(self.max_length):]
            prepared.append((ids, min(len(cont), len(ids) - 1)))
        order = sorted(range(len(prepared)), key=lambda i: len(prepared[i][0]))
        out: list = [None] * len(prepared)
        for b in range(0, len(order), self.batch_size):
            idx = order[b: b + self.batch_size]
            logits = self._logits_batch([prepared[i][0][:-1] for i in idx])
            for i, lg in zip(idx, logits):
                ids, n_cont = prepared[i]
                lp = torch.log_softmax(lg[-n_cont:], -1)
                tgt = torch.tensor(ids[-n_cont:], device=lp.device)
                out[i] = (float(lp.gather(-1, tgt[:, None]).sum()), bool((lp.argmax(-1) == tgt).all()))
        return out

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
        pairs = [((self.tok.encode(context) if context else [self.tok.eos_id]), self.tok.encode(continuation))
                 for context, continuation in requests]
        if self.batch_size == 1:
            return [self._score(c, k) for c, k in pairs]
        return self._score_many(pairs)

    def loglikelihood_rolling(self, texts) -> list[float]:
        chunks, owner = [], []
        for t, text in enumerate(texts):
            ids = [self.tok.eos_id] + self.tok.encode(text)
            for b in range(0, len(ids) - 1, self.max_length):
                chunk = ids[b: b + self.max_length + 1]
                chunks.append((chunk[:1], chunk[1:]))
                owner.append(t)
        scores = [self._score(c, k) for c, k in chunks] if self.batch_size == 1 else self._score_many(chunks)
        out = [0.0] * len(texts)
        for t, (lp, _) in zip(owner, scores):
            out[t] += lp
        return out

    @torch.no_grad()
    def _generate_lockstep(self, requests, max_new_tokens: int) -> list[str]:
        """Greedy decoding of several requests at once: every round runs all unfinished rows in one forward pass (right-
        padded; each row's next token is read at its own last position) and appends one token per row."""
        rows = [self.tok.encode(c) or [self.tok.eos_id] for c, _ in requests]
        new: list[list[int]] = [[] for _ in requests]
        live = list(range(len(requests)))
        for _ in range(max_new_tokens):
            if not live:
                break
            logits = self._logits_batch([(rows[i] + new[i])[-self.max_length:] for i in live])
            still = []
            for i, lg in zip(live, logits):
                nxt = int(lg[-1].argmax())
                if nxt == self.tok.eos_id:
                    continue
                new[i].append(nxt)
                text = self.tok.decode(new[i])
                if not any(s in text for s in (requests[i][1] or [])):
                    still.append(i)
            live = still
        out = []
        for i, (_, stops) in enumerate(requests):
            text = self.tok.decode(new[i])
            for s in (stops or []):
                text = text.split(s)[0]
            out.append(text)
        return out

    @torch.no_grad()
    def generate_until(self, requests, max_new_tokens: int = 64) -> list[str]:
        requests = list(requests)
        if self.batch_size > 1 and len(requests) > 1:
            out: list[str] = []
            for b in range(0, len(requests), self.batch_size):
                out += self._generate_lockstep(requests[b: b + self.batch_size], max_new_tokens)
            return out
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
