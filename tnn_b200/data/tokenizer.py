"""Decode-only GPT-2 vocabulary (``vocab.bin`` = u32 count, then (u32 length, bytes) per token;
reference: include/tokenizer/tokenizer.hpp:11-53, writer python/export_vocab.py)."""
from __future__ import annotations

import struct
from typing import Iterable, List

from ..host import H


class Tokenizer:
    def __init__(self, path: str):
        self._t = H.Tokenizer(path)

    def __len__(self):
        return len(self._t)

    def decode(self, ids: Iterable[int]) -> str:
        return self._t.decode([int(i) for i in ids]).decode("utf-8", errors="replace")

    def token_bytes(self, i: int) -> bytes:
        return self._t.token(int(i))


def write_vocab(path: str, tokens: List[bytes]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(tokens)))
        for t in tokens:
            f.write(struct.pack("<I", len(t)))
            f.write(t)
