"""Tokenizers for the tools, the evaluation tracks and the server: the Hugging Face tokenizer of the training data
when its files are available locally, a byte tokenizer otherwise (no network is assumed anywhere)."""
from __future__ import annotations

from typing import Any, Optional


class ByteTokenizer:
    """Fallback tokenizer (UTF-8 bytes + BOS/EOS) used when no Hugging Face tokenizer files are
    available offline.  ids 0..255 are bytes, 256 = BOS, 257 = EOS."""

    bos_token_id, eos_token_id, vocab_size = 256, 257, 258
    name = "bytes"

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


def load_tokenizer(name: Optional[str]) -> Any:
    """Hugging Face tokenizer from local files when present (the reference uses
    ``HuggingFaceTB/SmolLM2-135M``, ``serve.py:227-230``); the byte tokenizer otherwise."""
    if name:
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(name, local_files_only=True)
        except Exception:       # noqa: BLE001 - no network / no files
            pass
    return ByteTokenizer()
