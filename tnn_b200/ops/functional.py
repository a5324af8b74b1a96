"""``torch.autograd`` bridges to the hand-written kernels, for code that lives in ordinary PyTorch modules.

The framework's own layers (``nn/layers.py``) call explicit forward / backward kernels and never touch autograd. These
functions expose the same kernels to a model written with ``torch.nn`` and trained with ``loss.backward()``: each is a
``torch.autograd.Function`` whose forward and backward are one or two kernel launches (tcgen05 GEMM with fused bias /
GELU epilogues, fused flash attention on the packed QKV matrix, layer norm with fused residual add, streaming softmax
cross-entropy). On CPU tensors the same calls run the plain-torch references in ``ops/raw.py``, so a module built on
them runs anywhere.

    y = F.linear(x, w, b)                       # x [..., K] @ w[N, K]^T + b, optional fused tanh-GELU
    h, s = F.add_layer_norm(x, delta, g, b)     # s = x + delta ; h = LN(s)
    o = F.causal_self_attention(qkv, heads)     # qkv [B, S, 3E] packed q | k | v
    l = F.cross_entropy(logits, labels)         # mean over rows

Gradients with respect to weights are returned in fp32 (accumulated by the kernels in fp32) and cast by autograd to
the parameter's dtype.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import raw
from .gemm import gemm


def _flat2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1])


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, gelu):
        x2 = _flat2d(x).contiguous()
        z = torch.empty(x2.shape[0], w.shape[0], dtype=x2.dtype, device=x2.device) if gelu else None
        y = gemm(x2, w, bias=b, gelu=gelu, save_preact=z)
        ctx.save_for_backward(x2, w, z)
        ctx.has_bias, ctx.gelu, ctx.in_shape = b is not None, gelu, x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors
        dy2 = _flat2d(dy).contiguous()
        if ctx.gelu:  # back through the activation first: dz = dy * gelu'(z) from the saved pre-activation
            dy2 = raw.act_bwd(z, dy2, "gelu")
        dx = gemm(dy2, w, b_t=True).reshape(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1]:
            dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            gemm(dy2, x2, a_t=True, b_t=True, out=dw, atomic=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
            raw.colsum_accum(dy2, db)
        return dx, dw, db, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False) -> torch.Tensor:
    """``gelu(x @ weight.T + bias)`` with the bias and the tanh-GELU applied in the GEMM epilogue."""
    return _Linear.apply(x, weight, bias, gelu)


class _AddLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, gamma, beta, eps):
        x2 = _flat2d(x).contiguous()
        d2 = _flat2d(delta).contiguous() if delta is not None else None
        s, h, mean, rstd = raw.layernorm_fwd(x2, d2, gamma, beta, eps)
        s = x2 if s is None else s
        ctx.save_for_backward(s, mean, rstd, gamma)
        ctx.has_delta, ctx.shape = delta is not None, x.shape
        ctx.mark_non_differentiable(mean, rstd)
        return h.reshape(x.shape), s.reshape(x.shape)

    @staticmethod
    def backward(ctx, dh, ds):
        s, mean, rstd, gamma = ctx.saved_tensors
        C = s.shape[1]
        dg = torch.zeros(C, dtype=torch.float32, device=s.device) if gamma is not None else None
        db = torch.zeros(C, dtype=torch.float32, device=s.device) if gamma is not None else None
        dres = _flat2d(ds).contiguous() if ds is not None else None
        dx, _ = raw.layernorm_bwd(_flat2d(dh).contiguous(), s, mean, rstd, gamma, dres, False, 0.0, 0, dg, db)
        dx = dx.reshape(ctx.shape)
        return dx, (dx if ctx.has_delta else None), dg, db, None


def add_layer_norm(x: torch.Tensor, delta: Optional[torch.Tensor], gamma: Optional[torch.Tensor],
                   beta: Optional[torch.Tensor], eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """``s = x + delta`` (``delta`` may be None) and ``h = LayerNorm(s)`` over the last dimension in one pass.
    Returns ``(h, s)``: the pre-LN transformer block keeps ``s`` as its residual stream."""
    return _AddLayerNorm.apply(x, delta, gamma, beta, eps)


def layer_norm(x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    return _AddLayerNorm.apply(x, None, gamma, beta, eps)[0]


class _CausalSelfAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, heads, causal, scale):
        B, S, E3 = qkv.shape
        E = E3 // 3
        D = E // heads
        q2 = qkv.reshape(B * S, E3).contiguous()
        out, lse = raw.attn_fwd(q2, B, S, heads, D, causal, scale)
        ctx.save_for_backward(q2, out, lse)
        ctx.dims = (B, S, heads, D, causal, scale)
        return out.reshape(B, S, E)

    @staticmethod
    def backward(ctx, dout):
        q2, out, lse = ctx.saved_tensors
        B, S, H, D, causal, scale = ctx.dims
        dqkv = raw.attn_bwd(q2, out, dout.reshape(B * S, H * D).contiguous(), lse, B, S, H, D, causal, scale)
        return dqkv.reshape(B, S, 3 * H * D), None, None, None


def causal_self_attention(qkv: torch.Tensor, heads: int, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Flash attention on the packed projection ``qkv [B, S, 3E]`` (``q | k | v``, heads contiguous inside each):
    no head transposes, no score matrix in memory. ``scale`` defaults to ``1 / sqrt(head size)``."""
    D = qkv.shape[-1] // 3 // heads
    return _CausalSelfAttention.apply(qkv, heads, causal, float(scale) if scale is not None else D ** -0.5)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        l2 = _flat2d(logits)
        rows, vocab = l2.shape
        # the gradient of the mean loss is produced in the same pass and kept for backward
        loss, corrects, grad = raw.softmax_ce(l2, labels, vocab, 1.0 / rows, 1.0 / rows)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        ctx.mark_non_differentiable(corrects)
        return loss.reshape(()), corrects

    @staticmethod
    def backward(ctx, dloss, _):
        (grad,) = ctx.saved_tensors
        return (grad.float() * dloss).to(grad.dtype).reshape(ctx.shape), None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, return_corrects: bool = False):
    """Mean softmax cross-entropy over all rows of ``logits [..., V]`` with integer ``labels [...]``; with
    ``return_corrects`` also the number of rows whose arg-max equals the label (computed by the same kernel)."""
    loss, corrects = _CrossEntropy.apply(logits, labels)
    return (loss, corrects) if return_corrects else loss
