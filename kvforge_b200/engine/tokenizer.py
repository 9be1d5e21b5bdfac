"""Text in and out for demos with random weights.

The engine itself takes and returns token ids.  ``InferenceEngine`` accepts, for string prompts,
any object with ``encode(text) -> list[int]``, ``decode(ids) -> str`` and an ``eos_token_id``
attribute (``None`` if it has none); umarhassan-cloud/kvforge describes the same three as its
tokenizer protocol (src/tokenvault/model_loader.py:116-124).  ``BytesAsTokens`` is the one such
object that needs no vocabulary file.
"""

from __future__ import annotations


class BytesAsTokens:
    """The UTF-8 bytes of a text as token ids, fitted to the model's vocabulary.

    With 258 entries or more, ids 0 to 255 are the bytes, 256 opens a prompt and 257 is the
    end-of-sequence token (the numbering of kvforge's byte tokenizer, model_loader.py:127-137).
    A smaller vocabulary has no room for the two marks: prompts then start with their first
    byte and nothing ends a sequence but its length.  Below 256 entries bytes are folded into the
    vocabulary (``byte % vocab_size``), which loses the text but keeps a demo running.
    """

    def __init__(self, vocab_size: int = 258) -> None:
        if vocab_size < 1:
            raise ValueError("a vocabulary needs at least one entry")
        self.vocab_size = int(vocab_size)
        marks = self.vocab_size >= 258
        self.bos_token_id: int | None = 256 if marks else None
        self.eos_token_id: int | None = 257 if marks else None

    def encode(self, text: str) -> list[int]:
        data = text.encode("utf-8")
        ids = [b % self.vocab_size for b in data] if self.vocab_size < 256 else list(data)
        return ids if self.bos_token_id is None else [self.bos_token_id, *ids]

    def decode(self, token_ids: list[int]) -> str:
        return bytes(t for t in token_ids if 0 <= t < 256).decode("utf-8", errors="replace")


ByteTokenizer = BytesAsTokens  # the name kvforge uses
