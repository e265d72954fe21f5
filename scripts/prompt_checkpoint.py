#!/usr/bin/env python
"""Sample from a checkpoint: one prompt (--prompt) or an interactive loop. Temperature / top-k / top-p sampling with
a seeded generator; no KV cache (the prefix is re-run, padded to a multiple of 32)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def sample_next(logits, temperature, top_k, top_p, gen):
    import torch

    if temperature <= 0:
        return int(logits.argmax())
    logits = logits.float() / temperature
    if top_k:
        kth = torch.topk(logits, min(top_k, logits.numel())).values[-1]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = torch.softmax(logits, -1)
    if top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        keep = torch.cumsum(sp, 0) - sp < top_p
        probs = torch.zeros_like(probs).scatter(0, si[keep], sp[keep])
        probs = probs / probs.sum()
    return int(torch.multinomial(probs.cpu(), 1, generator=gen))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--prompt")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    import torch

    from open_transformers_b200.cli.eval import load_model_from_checkpoint
    from open_transformers_b200.data.tokenizer import Tokenizer

    model, cfg, _ = load_model_from_checkpoint(a.checkpoint, a.device)
    tok = Tokenizer(a.tokenizer)
    gen = torch.Generator().manual_seed(a.seed)

    def complete(prompt):
        ids = tok.encode(prompt) or [tok.eos_id]
        with torch.no_grad():
            for _ in range(a.max_new_tokens):
                ctx = ids[-cfg.train.seq_len:]
                pad = (-len(ctx)) % 32
                x = torch.tensor([ctx + [tok.eos_id] * pad], device=a.device)
                nxt = sample_next(model(x).logits[0, len(ctx) - 1], a.temperature, a.top_k, a.top_p, gen)
                if nxt == tok.eos_id:
                    break
                ids.append(nxt)
        return tok.decode(ids)

    if a.prompt is not None:
        print(complete(a.prompt))
        return
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        print(complete(line))


if __name__ == "__main__":
    main()
