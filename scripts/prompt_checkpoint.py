#!/usr/bin/env python3
"""Continue text from a checkpoint: one prompt (``--prompt``) or an interactive loop that streams tokens as they come.

    python scripts/prompt_checkpoint.py --checkpoint runs/<run>/checkpoints/step_<N> --tokenizer tokenizer.json [--prompt TEXT]

The model is a base model: give it the beginning of a text, not a question. The configuration comes from the checkpoint's
``meta.json`` (``--config-name`` / ``--override`` are accepted and ignored beyond a consistency note). There is no KV cache:
every new token re-runs the prefix, right-padded to a multiple of 32 positions.

Commands at the prompt (a line starting with ``:``):
    :temp X      sampling temperature (0 = greedy)
    :topk N      keep the N most likely tokens (0 = off)
    :topp P      nucleus sampling mass (1 = off)
    :tokens N    new tokens per continuation
    :seed N      reseed the sampler
    :show        current settings
    :help        this text
    :quit        leave (also Ctrl-D)
(reference scripts/prompt_checkpoint.py:43-218)
"""
from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@dataclass
class Settings:
    temperature: float = 0.8
    top_k: int = 50
    top_p: float = 0.95
    max_new_tokens: int = 200
    seed: int = 0

    def line(self) -> str:
        return "temperature=%g top_k=%d top_p=%g max_new_tokens=%d seed=%d" % (self.temperature, self.top_k, self.top_p, self.max_new_tokens, self.seed)


def sample_next(logits, s: Settings, gen) -> int:
    import torch

    if s.temperature <= 0:
        return int(logits.argmax())
    logits = logits.float() / s.temperature
    if s.top_k:
        kth = torch.topk(logits, min(s.top_k, logits.numel())).values[-1]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = torch.softmax(logits, -1)
    if s.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        keep = torch.cumsum(sp, 0) - sp < s.top_p
        probs = torch.zeros_like(probs).scatter(0, si[keep], sp[keep])
        probs = probs / probs.sum()
    return int(torch.multinomial(probs.cpu(), 1, generator=gen))


class Session:
    """Settings, sampler state and the command table of one interactive run."""

    def __init__(self, settings: Settings, out=sys.stdout):
        import torch

        self.s, self.out = settings, out
        self.gen = torch.Generator().manual_seed(settings.seed)
        # name -> (attribute, parser, lowest value allowed)
        self.setters = {"temp": ("temperature", float, 0.0), "topk": ("top_k", int, 0), "topp": ("top_p", float, 0.0), "tokens": ("max_new_tokens", int, 1)}

    def say(self, text: str) -> None:
        print(text, file=self.out)

    def command(self, line: str) -> bool:
        """True when `line` was a command (handled here), False when it is a prompt."""
        if not line.startswith(":"):
            return False
        name, *args = line[1:].split() or [""]
        if name in ("quit", "q", "exit"):
            raise SystemExit(0)
        if name in ("help", "h", "?"):
            self.say(__doc__)
        elif name == "show":
            self.say(self.s.line())
        elif name == "seed" and args:
            try:
                self.s.seed = int(args[0])
            except ValueError:
                self.say("not a number: %s" % args[0])
            else:
                self.gen.manual_seed(self.s.seed)
                self.say("seed = %d" % self.s.seed)
        elif name in self.setters and args:
            attr, parse, low = self.setters[name]
            try:
                value = parse(args[0])
            except ValueError:
                self.say("not a number: %s" % args[0])
            else:
                if value < low or (attr == "top_p" and value > 1.0):
                    self.say("%s out of range: %s" % (attr, args[0]))
                else:
                    setattr(self.s, attr, value)
                    self.say("%s = %s" % (attr, value))
        elif name in self.setters or name == "seed":
            self.say(":%s needs a value" % name)
        else:
            self.say("unknown command :%s (try :help)" % name)
        return True

    def complete(self, model, tok, prompt: str, device, max_seq_len: int, stream: bool = True) -> str:
        """Prints the prompt's continuation token by token (the text decoded so far is re-decoded each step, so multi-byte
        characters come out whole) and returns prompt + continuation."""
        import torch

        ids = tok.encode(prompt) or [tok.eos_id]
        shown = tok.decode(ids)
        if stream:
            self.out.write(shown)
            self.out.flush()
        with torch.no_grad():
            for _ in range(self.s.max_new_tokens):
                ctx = ids[-max_seq_len:]
                pad = (-len(ctx)) % 32
                x = torch.tensor([ctx + [tok.eos_id] * pad], device=device)
                nxt = sample_next(model(x).logits[0, len(ctx) - 1], self.s, self.gen)
                if nxt == tok.eos_id:
                    break
                ids.append(nxt)
                text = tok.decode(ids)
                if stream and not text.endswith("�"):
                    self.out.write(text[len(shown):])
                    self.out.flush()
                    shown = text
        text = tok.decode(ids)
        if stream:
            self.out.write(text[len(shown):] + "\n")
            self.out.flush()
        return text


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="prompt_checkpoint", description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint", required=True, help="checkpoint directory (with dcp/ and meta.json)")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--config-name", default=None, help="accepted for compatibility: the checkpoint's own configuration is used")
    ap.add_argument("--override", nargs="*", default=[])
    ap.add_argument("--device", default=None, help="cuda or cpu (default: cuda when there is one)")
    ap.add_argument("--dtype", choices=["bf16", "fp16", "fp32"], default="bf16",
                    help="accepted for compatibility: the forward pass runs in the precision the checkpoint's run trained in (its kernels "
                         "are bit-defined per precision family; there is no autocast to switch)")
    ap.add_argument("--prompt", help="continue this text once and exit")
    ap.add_argument("--max-new-tokens", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    import torch

    from open_transformers_b200.cli.eval import load_model_from_checkpoint
    from open_transformers_b200.data.tokenizer import Tokenizer

    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    print("loading %s on %s ..." % (a.checkpoint, device), file=sys.stderr)
    model, cfg, _ = load_model_from_checkpoint(a.checkpoint, device)
    tok = Tokenizer(a.tokenizer)
    print("%.2f B parameters, vocabulary %d, context %d" % (model.num_parameters() / 1e9, cfg.model.vocab_size, cfg.train.seq_len), file=sys.stderr)
    session = Session(Settings(a.temperature, a.top_k, a.top_p, a.max_new_tokens, a.seed))
    if a.prompt is not None:
        session.complete(model, tok, a.prompt, device, cfg.train.seq_len)
        return 0
    print("type the beginning of a text; :help lists the commands, :quit or Ctrl-D leaves\nsettings: " + session.s.line(), file=sys.stderr)
    while True:
        try:
            line = input("\n> ")
        except (EOFError, KeyboardInterrupt):
            print()
            return 0
        if not line.strip() or session.command(line.strip()):
            continue
        try:
            session.complete(model, tok, line, device, cfg.train.seq_len)
        except KeyboardInterrupt:
            print("\n[interrupted]")


if __name__ == "__main__":
    sys.exit(main())
