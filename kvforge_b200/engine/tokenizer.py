"""Tokenizer protocol and the dependency-free byte tokenizer for demos with random weights
(umarhassan-cloud/kvforge, src/tokenvault/model_loader.py:116-137).  The engine itself takes
and returns token ids; a tokenizer is only needed for string prompts."""

from __future__ import annotations

from typing import Protocol


class Tokenizer(Protocol):
    eos_token_id: int | None
    bos_token_id: int | None

    def encode(self, text: str) -> list[int]: ...

    def decode(self, token_ids: list[int]) -> str: ...


class ByteTokenizer:
    """UTF-8 bytes as tokens 0..255, BOS 256, EOS 257 (vocabulary 258)."""

    def __init__(self) -> None:
        self.bos_token_id = 256
        self.eos_token_id = 257
        self.vocab_size = 258

    def encode(self, text: str) -> list[int]:
        return [self.bos_token_id, *text.encode("utf-8")]

    def decode(self, token_ids: list[int]) -> str:
        return bytes(t for t in token_ids if 0 <= t < 256).decode("utf-8", errors="replace")
