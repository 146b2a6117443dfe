"""Byte-level stand-in tokenizer for the serving path. The reference serves text only through vLLM or a canned
mock (server/mock_engine.py:51-103) and has no tokenizer of its own; real checkpoints bring their Hugging Face
tokenizer, random-init models use this reversible byte mapping."""
from __future__ import annotations

from typing import List

_SYL = ["ka", "to", "mi", "ra", "ne", "so", "lu", "vi", "do", "pe", "ga", "xi", "bu", "zo", "he", "ny"]


class ByteTokenizer:
    def __init__(self, vocab: int):
        self.vocab = vocab

    def encode(self, text: str) -> List[int]:
        ids = [b % self.vocab for b in text.encode("utf-8")]
        return ids or [0]

    def piece(self, token: int) -> str:
        """Readable piece for any id: printable ASCII maps to itself, everything else to a syllable word."""
        if 32 <= token < 127:
            return chr(token)
        t, parts = token, []
        while True:
            parts.append(_SYL[t % 16])
            t //= 16
            if t == 0:
                break
        return " " + "".join(parts)

    def decode(self, tokens: List[int]) -> str:
        return "".join(self.piece(t) for t in tokens)


class HFTokenizer:
    """Thin wrapper over ``transformers.AutoTokenizer`` for real checkpoints."""

    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(path)

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text)

    def piece(self, token: int) -> str:
        return self.tok.decode([token])

    def decode(self, tokens: List[int]) -> str:
        return self.tok.decode(tokens)
