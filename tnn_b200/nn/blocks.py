"""Composite layers: ``sequential``, ``residual_block`` and ``flash_attention_block``.

Reference: src/nn/blocks_impl/{sequential,residual_block,flash_attention_block}.cpp.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops import raw
from ..ops.gemm import gemm
from .layers import (LAYER_REGISTRY, T_JSON, T_SIZE, T_STR, Conv2D, Layer, ParamSpec, _flat2d, register)


def layer_from_config(cfg: dict) -> Layer:
    t = cfg.get("type", "")
    if t not in LAYER_REGISTRY:
        raise ValueError(f"Unknown layer type: {t}")
    return LAYER_REGISTRY[t].from_config(cfg)


class _Composite(Layer):
    def children(self) -> List[Layer]:
        raise NotImplementedError

    def sublayers(self):
        return self.children()

    def param_specs(self):
        specs = []
        for c in self.children():
            specs += c.param_specs()
        return specs

    def bind(self, params, grads):
        super().bind(params, grads)
        i = 0
        for c in self.children():
            n = len(c.param_specs())
            c.bind(params[i:i + n], grads[i:i + n])
            i += n

    def bind_masters(self, masters):
        self.masters = masters
        i = 0
        for c in self.children():
            n = len(c.param_specs())
            c.bind_masters(masters[i:i + n])
            i += n

    def param_descriptors(self):
        out = []
        for c in self.children():
            out += c.param_descriptors() if hasattr(c, "param_descriptors") else list(c.params)
        return out


@register
class Sequential(_Composite):
    TYPE_NAME = "sequential"

    def __init__(self, layers: Optional[List[Layer]] = None, name: str = ""):
        super().__init__(name)
        self.layers: List[Layer] = list(layers or [])

    def children(self):
        return self.layers

    def config_items(self):
        return [("layers", T_JSON, [l.get_config() for l in self.layers])]

    @classmethod
    def from_config(cls, cfg):
        subs = cfg.get("parameters", {}).get("layers", {}).get("value", [])
        return cls([layer_from_config(c) for c in subs], name=cfg.get("name", ""))

    def output_shape(self, in_shapes):
        s = tuple(in_shapes[0])
        for l in self.layers:
            s = l.output_shape([s])
        return s

    def forward(self, inputs, ctx):
        x = inputs[0]
        for i, l in enumerate(self.layers):
            sub = ctx.setdefault(i, {"_step": ctx.get("_step", 0), "_pid": ctx.get("_pid", 0)})
            x = l.forward([x], sub)
        return x

    def backward(self, grad, ctx):
        for i in reversed(range(len(self.layers))):
            grad = self.layers[i].backward(grad, ctx[i])[0]
        return [grad]


@register
class ResidualBlock(_Composite):
    """``act(main(x) + shortcut(x))``; an empty shortcut is the identity
    (src/nn/blocks_impl/residual_block.cpp:60-125)."""
    TYPE_NAME = "residual_block"

    def __init__(self, main_path: Optional[Sequential] = None, shortcut_path: Optional[Sequential] = None,
                 activation: str = "relu", name: str = ""):
        super().__init__(name)
        self.main = main_path if main_path is not None else Sequential([], name=self.name + "_main")
        self.shortcut = shortcut_path
        self.activation = activation or "none"

    def children(self):
        return [self.main] + ([self.shortcut] if self.shortcut is not None else [])

    def config_items(self):
        return [("activation", T_STR, self.activation), ("main_path", T_JSON, self.main.get_config()),
                ("shortcut_path", T_JSON, self.shortcut.get_config() if self.shortcut is not None else {})]

    @classmethod
    def from_config(cls, cfg):
        p = cfg.get("parameters", {})
        main = Sequential.from_config(p["main_path"]["value"])
        sc_cfg = p.get("shortcut_path", {}).get("value") or None
        sc = Sequential.from_config(sc_cfg) if sc_cfg else None
        return cls(main, sc, p.get("activation", {}).get("value", "relu"), name=cfg.get("name", ""))

    def output_shape(self, in_shapes):
        return self.main.output_shape(in_shapes)

    def forward(self, inputs, ctx):
        x = inputs[0]
        base = {"_step": ctx.get("_step", 0), "_pid": ctx.get("_pid", 0)}
        ctx["m"], ctx["s"] = dict(base), dict(base)
        if self._closing_add_in_batchnorm(x):
            # shortcut first; the main path's last batch norm adds it and applies the ReLU in its own pass
            s = self.shortcut.forward([x], ctx["s"]) if self.shortcut is not None else x
            ctx["m"][len(self.main.layers) - 1] = dict(base, _add_relu=s.contiguous())
            y = self.main.forward([x], ctx["m"])
            ctx["y"] = y
            return y
        m = self.main.forward([x], ctx["m"])
        s = self.shortcut.forward([x], ctx["s"]) if self.shortcut is not None else x
        if self.activation == "relu":
            y = raw.binary(m, s, "add", relu=True)
            ctx["y"] = y
            return y
        z = raw.binary(m, s, "add")
        if self.activation in ("none", "linear", ""):
            return z
        ctx["z"] = z
        return raw.act_fwd(z, self.activation, 1.0 if self.activation == "elu" else 0.01)

    def _closing_add_in_batchnorm(self, x) -> bool:
        from .layers import BatchNorm
        if self.activation != "relu" or not self.main.layers:
            return False
        last = self.main.layers[-1]
        return isinstance(last, BatchNorm) and not last.use_relu and x.dim() == 4

    def backward(self, grad, ctx):
        if self.activation == "relu":
            grad = raw.act_bwd(ctx["y"], grad, "relu")  # y > 0 <=> pre-activation > 0
        elif "z" in ctx:
            grad = raw.act_bwd(ctx["z"], grad, self.activation, 1.0 if self.activation == "elu" else 0.01)
        gs = self.shortcut.backward(grad, ctx["s"])[0] if self.shortcut is not None else grad
        first = self.main.layers[0] if self.main.layers else None
        if isinstance(first, Conv2D) and not ctx["m"][0].get("_skip_dgrad"):
            # the main path's first convolution adds the shortcut's gradient while it writes its own input gradient
            ctx["m"][0]["_add_to_dx"] = gs
            return [self.main.backward(grad, ctx["m"])[0]]
        gm = self.main.backward(grad, ctx["m"])[0]
        return [raw.binary(gm, gs, "add")]


@register
class FlashAttentionBlock(Layer):
    """Multi-head self-attention: q/k/v/out projections around flash attention.

    The reference block (src/nn/blocks_impl/flash_attention_block.cpp:39-138) runs four separate
    biased dense layers, three ``[B,S,H,D] -> [B,H,S,D]`` transposes, cuDNN SDPA with
    ``attn_scale = 1.0`` (``:61,153``) and a transpose back. Here q/k/v live in one ``[3E, E]``
    weight so the projection is a single GEMM whose packed output the attention kernel reads in
    place; there are no transposes. The checkpoint still sees the reference's eight tensors
    (q.W, q.b, k.W, k.b, v.W, v.b, out.W, out.b) through :meth:`param_descriptors`.
    ``is_causal`` is not part of the saved config (a reloaded block is causal), as in the reference.

    ``recompute_qkv`` (attribute, default off): do not keep the packed q/k/v projection for the backward pass but
    compute it again from the saved input - the reference's backward always does this
    (src/nn/blocks_impl/flash_attention_block.cpp:216-224); here it trades one extra GEMM per block for
    ``3 * B * S * E`` elements of saved activations. ``Graph.set_recompute_qkv`` switches every block of a model.
    """
    TYPE_NAME = "flash_attention_block"

    def __init__(self, embed_dim: int, num_heads: int, is_causal: bool = True, attn_scale: float = 1.0, name: str = ""):
        super().__init__(name)
        self.embed_dim, self.num_heads, self.is_causal = int(embed_dim), int(num_heads), bool(is_causal)
        if self.embed_dim % self.num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.head_dim = self.embed_dim // self.num_heads
        self.attn_scale = float(attn_scale)
        self.recompute_qkv = False

    def config_items(self):
        return [("embed_dim", T_SIZE, self.embed_dim), ("num_heads", T_SIZE, self.num_heads)]

    def param_specs(self):
        E = self.embed_dim
        std = 1.0 / math.sqrt(E)
        tp = getattr(self, "tp", 1)  # tensor parallelism: heads are split, q|k|v each [E/tp, E], out [E, E/tp]
        sh = tp > 1
        return [ParamSpec("qkv_weight", (3 * E // tp, E), True, ("normal", std), sharded=sh),
                ParamSpec("qkv_bias", (3 * E // tp,), True, ("normal", std), sharded=sh),
                ParamSpec("out_weight", (E, E // tp), True, ("normal", std), sharded=sh),
                ParamSpec("out_bias", (E,), True, ("normal", std))]

    def param_descriptors(self):
        E = self.embed_dim // getattr(self, "tp", 1)
        w, b, wo, bo = self.params
        return [w[0:E], b[0:E], w[E:2 * E], b[E:2 * E], w[2 * E:3 * E], b[2 * E:3 * E], wo, bo]

    def forward(self, inputs, ctx):
        x = inputs[0]
        B, S, E = x.shape
        x2 = _flat2d(x)
        w, b, wo, bo = self.params
        qkv = gemm(x2, w, bias=b, out_dtype=x.dtype)
        a, lse = raw.attn_fwd(qkv, B, S, self.num_heads, self.head_dim, self.is_causal, self.attn_scale)
        y = gemm(a, wo, bias=bo, out_dtype=x.dtype)
        ctx.update(x=x2, qkv=None if self.recompute_qkv else qkv, a=a, lse=lse, dims=(B, S))
        return y.reshape(B, S, E)

    def backward(self, grad, ctx):
        B, S = ctx["dims"]
        w, b, wo, bo = self.params
        dy = _flat2d(grad)
        if self.grads[0] is not None:
            gemm(dy, ctx["a"], a_t=True, b_t=True, out=self.grads[2], atomic=True)
            raw.colsum_accum(dy, self.grads[3])
        da = gemm(dy, wo, b_t=True, out_dtype=dy.dtype)
        qkv = ctx["qkv"] if ctx["qkv"] is not None else gemm(ctx["x"], w, bias=b, out_dtype=dy.dtype)
        dqkv = raw.attn_bwd(qkv, ctx["a"], da, ctx["lse"], B, S, self.num_heads, self.head_dim, self.is_causal,
                            self.attn_scale)
        if self.grads[0] is not None:
            gemm(dqkv, ctx["x"], a_t=True, b_t=True, out=self.grads[0], atomic=True)
            raw.colsum_accum(dqkv, self.grads[1])
        dx = gemm(dqkv, w, b_t=True, out_dtype=dy.dtype)
        return [dx.reshape(B, S, self.embed_dim)]
