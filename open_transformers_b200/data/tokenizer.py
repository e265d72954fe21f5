"""Byte-level BPE tokenizer (HF `tokenizers` backend): training, hashing, thin wrapper.

Training recipe: byte-fallback BPE, digits isolated one by one, GPT-2 style byte-level pre-tokenisation
without prefix space, 128 256 entries including six specials, of which ``<|endoftext|>`` is the document
separator (reference src/pretrain/data/tokenizer.py:25-141)."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Iterable

SPECIAL_TOKENS = ["<|endoftext|>", "<|begin_of_text|>", "<|start_header|>", "<|end_header|>", "<|eot|>", "<|pad|>"]


def train_tokenizer(text_iterator: Iterable[str], output_path: str | Path, vocab_size: int = 128_256, min_frequency: int = 2,
                    special_tokens: list[str] | None = None, show_progress: bool = False) -> Path:
    from tokenizers import Regex
    from tokenizers import Tokenizer as HFTokenizer
    from tokenizers import decoders, models, pre_tokenizers, processors, trainers

    out = Path(output_path)
    out.parent.mkdir(parents=True, exist_ok=True)
    tok = HFTokenizer(models.BPE(byte_fallback=True))
    # every digit its own piece (a Regex: a plain string pattern would be matched literally), then GPT-2 byte-level pieces
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(pattern=Regex(r"\d"), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)])
    tok.decoder = decoders.ByteLevel()
    tok.post_processor = processors.ByteLevel(trim_offsets=False)
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, min_frequency=min_frequency, special_tokens=special_tokens or SPECIAL_TOKENS,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=show_progress)
    tok.train_from_iterator(text_iterator, trainer=trainer)
    tmp = out.with_suffix(out.suffix + ".tmp")   # write-then-rename: a crash never leaves a half-written tokenizer
    tok.save(str(tmp))
    tmp.replace(out)
    return out


def compute_hash(path: str | Path) -> str:
    """sha256 of the tokenizer's canonical JSON (sorted keys, no whitespace): stable across re-serialisation."""
    data = json.loads(Path(path).read_text(encoding="utf-8"))
    return hashlib.sha256(json.dumps(data, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode("utf-8")).hexdigest()


class Tokenizer:
    def __init__(self, path: str | Path):
        from tokenizers import Tokenizer as HFTokenizer

        self.path = Path(path)
        self._tok = HFTokenizer.from_file(str(path))
        self.hash = compute_hash(path)
        eos = self._tok.token_to_id("<|endoftext|>")
        if eos is None:
            raise ValueError("%s has no <|endoftext|> token" % path)
        self.eos_id = int(eos)

    @property
    def vocab_size(self) -> int:
        return self._tok.get_vocab_size()

    def encode(self, text: str) -> list[int]:
        return self._tok.encode(text, add_special_tokens=False).ids

    def encode_batch(self, texts: list[str]) -> list[list[int]]:
        return [e.ids for e in self._tok.encode_batch(texts, add_special_tokens=False)]

    def decode(self, ids) -> str:
        return self._tok.decode(list(int(i) for i in ids), skip_special_tokens=False)

    def decode_batch(self, batch, skip_special_tokens: bool = False) -> list[str]:
        """Several id sequences at once (special tokens kept by default, so the text stays faithful to the stored ids)."""
        return self._tok.decode_batch([[int(i) for i in ids] for ids in batch], skip_special_tokens=skip_special_tokens)
