"""Inference helpers: validation of a saved or fresh model and greedy text generation.

Reference: examples/inferencer.cpp:12-70 (validation loss / accuracy from ``model_path`` or a fresh zoo
model) and examples/gpt2_inference.cpp:16-114 (greedy decoding: the prompt is right-padded with zeros to
the model's sequence length, the logits at the last real position pick the next token, decoding stops
at token 50256).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional

import torch

from .nn.graph import Graph
from .nn.layers import PositionalEmbedding


def model_seq_len(graph: Graph) -> Optional[int]:
    """Sequence length fixed by the positional embedding of a language model (None if there is none)."""
    for layer in graph.layers():
        if isinstance(layer, PositionalEmbedding):
            return int(layer.seq_len)
    return None


@torch.no_grad()
def greedy_generate(graph: Graph, prompt: Iterable[int], num_new: int = 50, eos: Optional[int] = 50256,
                    seq_len: Optional[int] = None, on_token: Optional[Callable[[int], None]] = None) -> List[int]:
    """Greedy decoding with a full forward pass per token (the reference has no KV cache either).

    ``seq_len`` defaults to the model's positional-embedding length; the window slides once the text is
    longer than that. Returns prompt + generated tokens.
    """
    tokens = [int(t) for t in prompt]
    if not tokens:
        raise ValueError("empty prompt")
    S = seq_len or model_seq_len(graph) or len(tokens) + num_new
    was_training = graph.training
    graph.set_training(False)
    try:
        for _ in range(num_new):
            use = tokens[-S:]
            x = torch.zeros(1, S, dtype=torch.long)
            x[0, :len(use)] = torch.tensor(use)
            out = graph.forward({graph.input_nodes[0].uid(): x.to(graph.device)})[graph.output_nodes[0].uid()]
            logits = out[0, len(use) - 1].float()
            if bool(torch.isnan(logits[0])):
                raise FloatingPointError("model output contains NaNs (the model probably diverged in training)")
            nxt = int(torch.argmax(logits))
            tokens.append(nxt)
            if on_token is not None:
                on_token(nxt)
            if eos is not None and nxt == eos:
                break
    finally:
        graph.set_training(was_training)
    return tokens


@torch.no_grad()
def evaluate(trainer, max_batches: Optional[int] = None) -> Dict[str, float]:
    """Validation loss / accuracy (and perplexity for token models) through the trainer's own loop."""
    return dict(trainer.validate(max_batches=max_batches))
