"""Prepare a token corpus for the ``open_webtext`` loader: ``train.bin`` / ``val.bin`` (flat uint16 ids) and ``vocab.bin``.

    python -m tnn_b200.data.prepare_text --out data/open-web-text --input corpus/*.txt [--tokenizer gpt2|bytes] [--val-fraction 0.0005]

The reference prepares OpenWebText with ``python/openwebtext.py`` (tiktoken GPT-2 encoding, every document followed by
the end-of-text id, ids written as uint16) and ``python/export_vocab.py`` (``vocab.bin`` = u32 count, then u32 length +
bytes per token). This does the same for local text files. ``--tokenizer gpt2`` uses tiktoken when it is installed,
else a GPT-2 tokenizer of ``transformers`` found in the local cache; ``--tokenizer bytes`` (no dependency: ids 0-255 are
the bytes, 256 is end-of-text) keeps the pipeline usable on a machine without either - the decode-only
``Tokenizer`` reads its ``vocab.bin`` like any other.
"""
from __future__ import annotations

import argparse
import glob
import os
from typing import Callable, List, Tuple

import numpy as np

from .tokenizer import write_vocab


def byte_tokenizer() -> Tuple[Callable[[str], List[int]], int, List[bytes]]:
    vocab = [bytes([i]) for i in range(256)] + [b"<|endoftext|>"]
    return (lambda text: list(text.encode("utf-8"))), 256, vocab


def gpt2_tokenizer() -> Tuple[Callable[[str], List[int]], int, List[bytes]]:
    try:
        import tiktoken

        enc = tiktoken.get_encoding("gpt2")
        vocab = [enc.decode_single_token_bytes(i) for i in range(enc.n_vocab)]
        return enc.encode_ordinary, enc.eot_token, vocab
    except Exception:
        pass
    from transformers import GPT2TokenizerFast

    tok = GPT2TokenizerFast.from_pretrained("gpt2", local_files_only=True)
    byte_decoder = {c: b for b, c in _bytes_to_unicode().items()}
    vocab = [b""] * len(tok)
    for s, i in tok.get_vocab().items():
        vocab[i] = bytes(byte_decoder.get(ch, ord("?")) for ch in s)
    return (lambda text: tok.encode(text, add_special_tokens=False)), tok.eos_token_id, vocab


def _bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, (chr(c) for c in cs)))


def prepare(inputs: List[str], out_dir: str, tokenizer: str = "gpt2", val_fraction: float = 0.0005, paragraph_docs: bool = False) -> dict:
    encode, eot, vocab = byte_tokenizer() if tokenizer == "bytes" else gpt2_tokenizer()
    if len(vocab) > 65536:
        raise ValueError("the token files are uint16: the vocabulary must have at most 65536 entries")
    os.makedirs(out_dir, exist_ok=True)
    docs: List[str] = []
    for path in inputs:
        with open(path, "r", encoding="utf-8", errors="replace") as f:
            text = f.read()
        docs += [d for d in text.split("\n\n") if d.strip()] if paragraph_docs else [text]
    n_val = max(1, int(round(len(docs) * val_fraction))) if len(docs) > 1 else 0
    splits = {"val": docs[:n_val], "train": docs[n_val:]}
    counts = {}
    for name, ds in splits.items():
        with open(os.path.join(out_dir, f"{name}.bin"), "wb") as f:
            total = 0
            for d in ds:
                ids = np.asarray(encode(d) + [eot], dtype=np.uint16)  # every document ends with end-of-text
                f.write(ids.tobytes())
                total += len(ids)
        counts[name] = total
    write_vocab(os.path.join(out_dir, "vocab.bin"), vocab)
    return {"tokens": counts, "vocab": len(vocab), "eot": eot, "out": out_dir}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input", nargs="+", required=True, help="text files (globs allowed)")
    ap.add_argument("--out", default="data/open-web-text")
    ap.add_argument("--tokenizer", default="gpt2", choices=["gpt2", "bytes"])
    ap.add_argument("--val-fraction", type=float, default=0.0005)
    ap.add_argument("--paragraph-docs", action="store_true", help="treat blank-line separated paragraphs as documents")
    a = ap.parse_args(argv)
    files = sorted(p for pat in a.input for p in glob.glob(pat))
    if not files:
        raise SystemExit("no input files")
    print(prepare(files, a.out, a.tokenizer, a.val_fraction, a.paragraph_docs))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
