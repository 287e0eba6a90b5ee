"""Tokenizers: a byte-level fallback (vocab 256), a wrapper over Hugging Face ``tokenizers`` BPE files, and a BPE
trainer that reserves the chat / tool / ``<CARRY>`` special tokens (reference ``loomformer.py:1148-1239``)."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

SPECIAL_TOKENS = ["<pad>", "<bos>", "<eos>", "<|im_start|>", "<|im_end|>", "<think>", "</think>",
                  "<tool_call>", "</tool_call>", "<tool_response>", "</tool_response>", "<CARRY>"]


class ByteTokenizer:
    vocab_size = 256

    def encode(self, s: str) -> List[int]:
        return list(s.encode("utf-8"))

    def encode_batch(self, texts: List[str]) -> List[List[int]]:
        return [list(t.encode("utf-8")) for t in texts]

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")

    def special_id(self, token: str) -> Optional[int]:
        return None


class BPETokenizer:
    """Thin adapter over a ``tokenizers.Tokenizer``."""

    def __init__(self, tk) -> None:
        self.tk = tk
        self.vocab_size = tk.get_vocab_size()

    @classmethod
    def load(cls, path: str) -> "BPETokenizer":
        from tokenizers import Tokenizer
        return cls(Tokenizer.from_file(path))

    @classmethod
    def from_json_bytes(cls, blob: bytes) -> "BPETokenizer":
        from tokenizers import Tokenizer
        return cls(Tokenizer.from_str(blob.decode("utf-8")))

    def encode(self, s: str) -> List[int]:
        return self.tk.encode(s).ids

    def encode_batch(self, texts: List[str]) -> List[List[int]]:
        return [e.ids for e in self.tk.encode_batch(texts)]

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return self.tk.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def special_id(self, token: str) -> Optional[int]:
        return self.tk.token_to_id(token)


class HFTokenizer:
    """Adapter over a ``transformers`` tokenizer (name or local directory)."""

    def __init__(self, name: str) -> None:
        from transformers import AutoTokenizer
        self.tk = AutoTokenizer.from_pretrained(name)
        self.vocab_size = self.tk.vocab_size

    def encode(self, s: str) -> List[int]:
        return self.tk.encode(s, add_special_tokens=False)

    def encode_batch(self, texts: List[str]) -> List[List[int]]:
        return self.tk(texts, add_special_tokens=False)["input_ids"]

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return self.tk.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def special_id(self, token: str) -> Optional[int]:
        i = self.tk.convert_tokens_to_ids(token)
        return None if i is None or i == self.tk.unk_token_id else int(i)


def special_id(tok, name: str) -> Optional[int]:
    fn = getattr(tok, "special_id", None)
    return fn(name) if fn is not None else None


def build_tokenizer(cfg) -> Tuple[object, Optional[int]]:
    """Instantiate the tokenizer named by ``cfg.tokenizer`` (``None`` -> bytes), set ``cfg.vocab`` to its size and
    return ``(tokenizer, carry_token_id)``."""
    if cfg.tokenizer:
        if cfg.tokenizer.endswith(".json") and os.path.exists(cfg.tokenizer):
            tok = BPETokenizer.load(cfg.tokenizer)
        else:
            tok = HFTokenizer(cfg.tokenizer)
        cfg.vocab = tok.vocab_size
        return tok, special_id(tok, "<CARRY>")
    cfg.vocab = ByteTokenizer.vocab_size
    return ByteTokenizer(), None


def train_tokenizer(raw_dir: str, vocab_size: int, out: str, special_tokens: Optional[List[str]] = None,
                    dataset_format: str = "auto", text_field: str = "text", texts=None) -> None:
    """Train a byte-level BPE tokenizer on a raw corpus (or an explicit iterable of texts) and save it as JSON."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tk = Tokenizer(models.BPE(unk_token=None))
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    specials = list(SPECIAL_TOKENS if special_tokens is None else special_tokens)
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                  special_tokens=specials, show_progress=False)
    if texts is None:
        from .corpus import RawCorpus
        corpus = RawCorpus(raw_dir, fmt=str(dataset_format or "auto").lower(), text_field=text_field)
        tk.train_from_iterator(corpus.iter_texts(), trainer=trainer, length=len(corpus))
        note = f"format={corpus.fmt} docs={len(corpus)}"
    else:
        tk.train_from_iterator(iter(texts), trainer=trainer)
        note = "in-memory texts"
    tk.save(out)
    print(f"[train-tokenizer] vocab={tk.get_vocab_size()} {note} text_field={text_field!r} "
          f"special_tokens={specials} -> {out}")
