"""A GPT-2 style block written as an ordinary ``torch.nn.Module`` on top of ``tnn_b200.ops.functional`` and trained with
``loss.backward()`` and a stock ``torch.optim`` optimizer. On a B200 every call below is one of this framework's
kernels (tcgen05 GEMM with bias / GELU epilogue, fused add + layer norm, flash attention on the packed QKV matrix,
streaming softmax cross-entropy); on the CPU the same module runs on the plain-torch references.

    python examples/torch_module_with_kernels.py [--device cuda] [--steps 30]

The reference has no counterpart: its layers are only reachable through its own graph executor.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.ops import functional as F  # noqa: E402


class Block(torch.nn.Module):
    def __init__(self, embed: int, heads: int):
        super().__init__()
        mk = lambda *s, sc=0.02: torch.nn.Parameter(torch.randn(*s) * sc)
        self.heads = heads
        self.g1, self.b1 = torch.nn.Parameter(torch.ones(embed)), torch.nn.Parameter(torch.zeros(embed))
        self.g2, self.b2 = torch.nn.Parameter(torch.ones(embed)), torch.nn.Parameter(torch.zeros(embed))
        self.wqkv, self.bqkv = mk(3 * embed, embed), torch.nn.Parameter(torch.zeros(3 * embed))
        self.wo, self.bo = mk(embed, embed), torch.nn.Parameter(torch.zeros(embed))
        self.w1, self.bb1 = mk(4 * embed, embed), torch.nn.Parameter(torch.zeros(4 * embed))
        self.w2, self.bb2 = mk(embed, 4 * embed), torch.nn.Parameter(torch.zeros(embed))

    def forward(self, x, pending=None):
        """``pending`` is the previous block's MLP output, not yet added to the residual stream: the add is fused
        into this block's first layer norm."""
        h, x = F.add_layer_norm(x, pending, self.g1, self.b1)
        a = F.linear(F.causal_self_attention(F.linear(h, self.wqkv, self.bqkv), self.heads), self.wo, self.bo)
        h, x = F.add_layer_norm(x, a, self.g2, self.b2)
        return x, F.linear(F.linear(h, self.w1, self.bb1, gelu=True), self.w2, self.bb2)


class TinyGPT(torch.nn.Module):
    def __init__(self, vocab=64, seq=128, embed=64, heads=1, layers=2):
        super().__init__()
        self.wte, self.wpe = torch.nn.Embedding(vocab, embed), torch.nn.Embedding(seq, embed)
        self.blocks = torch.nn.ModuleList(Block(embed, heads) for _ in range(layers))
        self.gf, self.bf = torch.nn.Parameter(torch.ones(embed)), torch.nn.Parameter(torch.zeros(embed))
        self.head = torch.nn.Parameter(torch.randn(vocab, embed) * 0.02)

    def forward(self, ids, labels):
        x = self.wte(ids) + self.wpe(torch.arange(ids.shape[1], device=ids.device))
        pending = None
        for b in self.blocks:
            x, pending = b(x, pending)
        h, _ = F.add_layer_norm(x, pending, self.gf, self.bf)
        return F.cross_entropy(F.linear(h, self.head), labels)


def main(device="cpu", steps=30, seed=0):
    torch.manual_seed(seed)
    model = TinyGPT().to(device)
    if device != "cpu":
        model = model.to(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    seq = torch.randint(0, 64, (4, 129), device=device)
    ids, labels = seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
    first = last = None
    for step in range(steps):
        loss = model(ids, labels)
        opt.zero_grad()
        loss.backward()
        opt.step()
        last = float(loss.detach())
        first = last if first is None else first
        if step % 10 == 0:
            print(f"step {step} loss {last:.4f}")
    print(f"loss {first:.4f} -> {last:.4f}")
    return first, last


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=30)
    a = ap.parse_args()
    main(a.device, a.steps)
