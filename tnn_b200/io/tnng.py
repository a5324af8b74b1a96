"""TNNG graph-state files (reference: src/nn/graph.cpp:422-692) through the C++ codec.

A *state* is the plain dict produced by ``Graph.state()``: ``nodes`` (uids), ``inputs`` /
``outputs`` (node indices), ``layers`` (TConfig JSON text per unique layer), ``edges``
``(layer, producers, consumers)`` and ``params`` (per layer, tensors in descriptor order).
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from ..host import H

# dtype codes of the format (include/type/type.hpp:115-128)
CODES = {torch.uint8: 1, torch.int8: 2, torch.bool: 3, torch.float16: 4, torch.bfloat16: 5, torch.float32: 6,
         torch.float64: 7, torch.int32: 8, torch.int64: 9}
DTYPES = {v: k for k, v in CODES.items()}
DTYPES[0] = torch.uint8
DTYPES[10] = torch.int64


def tensor_to_record(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
    return (CODES[t.dtype], list(t.shape), raw)


def record_to_tensor(rec) -> torch.Tensor:
    code, shape, raw = rec
    dt = DTYPES[code]
    if len(raw) == 0:
        return torch.empty(shape, dtype=dt)
    flat = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy())
    return flat.view(dt).reshape(shape)


def _encode(state: dict) -> dict:
    d = dict(state)
    d["layers"] = [H.tconfig_normalize(s) for s in state["layers"]]
    d["edges"] = [tuple(e) for e in state["edges"]]
    d["params"] = [[tensor_to_record(t) for t in lp] for lp in state["params"]]
    return d


def _decode(d: dict) -> dict:
    d = dict(d)
    d["edges"] = [(int(l), list(p), list(c)) for (l, p, c) in d["edges"]]
    d["params"] = [[record_to_tensor(r) for r in lp] for lp in d["params"]]
    return d


def serialize(state: dict) -> bytes:
    return H.tnng_serialize(_encode(state))


def parse(data: bytes) -> dict:
    return _decode(H.tnng_parse(data))


def write_file(path: str, state: dict) -> None:
    H.tnng_write_file(path, _encode(state))


def read_file(path: str) -> dict:
    return _decode(H.tnng_read_file(path))


def save_tensor(t: torch.Tensor) -> bytes:
    """Raw tensor record: u32 dtype, u64 ndim, dims, bytes (include/tensor/tensor_ops.hpp:17-40)."""
    return H.tensor_serialize(tensor_to_record(t))


def load_tensor(data: bytes) -> torch.Tensor:
    return record_to_tensor(H.tensor_parse(data))
