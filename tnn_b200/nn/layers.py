"""Layer zoo with explicit forward / backward (no autograd tape).

Every layer mirrors one of the reference's registered layer types
(include/nn/layer_factory.hpp:65-132): same ``type`` string, same typed config
keys (src/nn/layers_impl/*.cpp ``get_config``), same parameter order
(``param_descriptors``) and the same semantics as the reference CPU engine
(src/nn/engines/cpu_engine.cpp). Activations are channels-last (NHWC images,
``[B, S, E]`` sequences); conv weights are ``[O, KH, KW, I]``, dense weights
``[out, in]``.

A layer owns no storage: ``Graph.compile`` allocates one flat parameter buffer,
one flat fp32 gradient buffer and (for bf16 training) one fp32 master buffer and
hands each layer views into them (``bind``). ``forward`` stores what the
backward needs in the per-micro-batch ``ctx`` dict - the counterpart of the
reference's ``Residuals`` keyed by ``pid`` (include/nn/layer.hpp:50-95) - so
several micro-batches can be in flight in one pipeline stage. ``backward``
accumulates parameter gradients (``+=``) and returns input gradients.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import raw
from ..ops.gemm import gemm

# TConfig value tags (src/common/config.cpp:86-130); size_t serialises as "unsigned long" on LP64.
T_SIZE, T_INT, T_FLOAT, T_BOOL, T_STR, T_JSON = "unsigned long", "int", "float", "bool", "string", "json"

LAYER_REGISTRY: Dict[str, type] = {}


def register(cls):
    LAYER_REGISTRY[cls.TYPE_NAME] = cls
    return cls


def f32(x: float) -> float:
    """Round to float32 the way a C++ ``float`` member would hold it."""
    return float(torch.tensor(x, dtype=torch.float32).item())


class ParamSpec:
    __slots__ = ("name", "shape", "trainable", "init", "sharded")

    def __init__(self, name: str, shape: Sequence[int], trainable: bool = True, init: Tuple[str, float] = ("zeros", 0.0),
                 sharded: bool = False):
        self.name, self.shape, self.trainable, self.init = name, tuple(int(s) for s in shape), trainable, init
        self.sharded = sharded  # True: this rank holds one tensor-parallel shard of the full parameter


class Layer:
    """Base class: config round-trip, parameter binding, explicit fwd/bwd."""

    TYPE_NAME = "layer"
    n_inputs = 1

    def __init__(self, name: str = ""):
        self.name = name or self.TYPE_NAME
        self.params: List[torch.Tensor] = []     # compute-dtype views, descriptor order
        self.grads: List[Optional[torch.Tensor]] = []  # fp32 views (None for non-trainable)
        self.training = True
        self.io_dtype = torch.float32
        self.seed_base = 0

    # ---- configuration ------------------------------------------------------------
    def config_items(self) -> List[Tuple[str, str, object]]:
        return []

    def get_config(self) -> dict:
        return {"name": self.name, "type": self.TYPE_NAME,
                "parameters": {k: {"type": t, "value": v} for k, t, v in self.config_items()}}

    @classmethod
    def from_config(cls, cfg: dict) -> "Layer":
        kw = {k: v["value"] for k, v in cfg.get("parameters", {}).items()}
        return cls(name=cfg.get("name", ""), **kw)

    # ---- parameters ---------------------------------------------------------------
    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, params: List[torch.Tensor], grads: List[Optional[torch.Tensor]]):
        self.params, self.grads = params, grads

    def bind_masters(self, masters: List[torch.Tensor]):
        self.masters = masters

    def sublayers(self) -> List["Layer"]:
        return []

    def set_training(self, flag: bool):
        self.training = flag
        for s in self.sublayers():
            s.set_training(flag)

    def set_io_dtype(self, dt: torch.dtype):
        self.io_dtype = dt
        for s in self.sublayers():
            s.set_io_dtype(dt)

    # ---- shapes / execution -------------------------------------------------------
    def output_shape(self, in_shapes: List[Tuple[int, ...]]) -> Tuple[int, ...]:
        return tuple(in_shapes[0])

    def forward(self, inputs: List[torch.Tensor], ctx: dict) -> torch.Tensor:
        raise NotImplementedError

    def backward(self, grad: torch.Tensor, ctx: dict) -> List[torch.Tensor]:
        raise NotImplementedError

    def step_seed(self, ctx: dict) -> int:
        """Dropout seed: unique per (layer, step, micro-batch), reproducible in backward."""
        return (hash(self.name) & 0xFFFFFFFF) * 1000003 + int(ctx.get("_step", 0)) * 7919 + int(ctx.get("_pid", 0)) * 104729 + self.seed_base


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


# ----------------------------------------------------------------------------- dense
@register
class Dense(Layer):
    """``Y = X W^T (+ b)``; reference: src/nn/layers_impl/dense_layer.cpp (which never adds the bias
    on its GPU engines because DenseStats.use_bias is left false - here the bias is applied)."""

    TYPE_NAME = "dense"

    def __init__(self, input_features: int, output_features: int, use_bias: bool = True, name: str = ""):
        super().__init__(name)
        self.input_features, self.output_features, self.use_bias = int(input_features), int(output_features), bool(use_bias)

    def config_items(self):
        return [("input_features", T_SIZE, self.input_features), ("output_features", T_SIZE, self.output_features),
                ("use_bias", T_BOOL, self.use_bias)]

    def param_specs(self):
        std = 1.0 / math.sqrt(self.input_features)
        # tensor parallelism (set by tnn_b200.parallel.tp): "col" splits the output features (weight
        # rows and bias), "row" splits the input features (weight columns; the bias stays replicated)
        tp, mode = getattr(self, "tp", 1), getattr(self, "tp_mode", None)
        out_f = self.output_features // tp if mode == "col" else self.output_features
        in_f = self.input_features // tp if mode == "row" else self.input_features
        specs = [ParamSpec("weight", (out_f, in_f), True, ("normal", std), sharded=mode is not None)]
        if self.use_bias:
            specs.append(ParamSpec("bias", (out_f,), True, ("normal", std), sharded=mode == "col"))
        return specs

    def output_shape(self, in_shapes):
        return tuple(in_shapes[0][:-1]) + (self.output_features,)

    def forward(self, inputs, ctx):
        x = inputs[0]
        x2 = _flat2d(x)
        ctx["x"] = x2
        ctx["shape"] = x.shape
        out = None
        n = self.output_features
        if x.is_cuda and n % 64:
            # Odd widths (a 50257-entry vocabulary) get a row pitch padded to 64 elements so that the
            # GEMM epilogue and the loss kernel keep their 16-byte vector path; callers see a view.
            out = torch.empty(x2.shape[0], (n + 63) // 64 * 64, dtype=x.dtype, device=x.device)[:, :n]
        y = gemm(x2, self.params[0], bias=self.params[1] if self.use_bias else None, out=out, out_dtype=x.dtype)
        return y.view(*x.shape[:-1], n)

    def backward(self, grad, ctx):
        dy = _flat2d(grad)
        x2 = ctx["x"]
        if self.grads[0] is not None:
            gemm(dy, x2, a_t=True, b_t=True, out=self.grads[0], atomic=True)
            if self.use_bias:
                raw.colsum_accum(dy, self.grads[1])
        dx = gemm(dy, self.params[0], b_t=True, out_dtype=dy.dtype)
        return [dx.reshape(ctx["shape"])]


@register
class LegacyDense(Dense):
    TYPE_NAME = "legacy_dense"


# ----------------------------------------------------------------------- activations
class _Activation(Layer):
    KIND = "linear"

    def __init__(self, name: str = ""):
        super().__init__(name)
        self.alpha = 0.0

    def forward(self, inputs, ctx):
        ctx["x"] = inputs[0]
        return raw.act_fwd(inputs[0], self.KIND, self.alpha)

    def backward(self, grad, ctx):
        return [raw.act_bwd(ctx["x"], grad, self.KIND, self.alpha)]


@register
class ReLU(_Activation):
    TYPE_NAME, KIND = "relu", "relu"


@register
class GELU(_Activation):
    """tanh-form GELU (src/nn/activations_impl/cuda/gelu_kernels.cu:18-59)."""
    TYPE_NAME, KIND = "gelu", "gelu"


@register
class Sigmoid(_Activation):
    TYPE_NAME, KIND = "sigmoid", "sigmoid"


@register
class Tanh(_Activation):
    TYPE_NAME, KIND = "tanh", "tanh"


@register
class Linear(_Activation):
    TYPE_NAME, KIND = "linear", "linear"


@register
class ELU(_Activation):
    TYPE_NAME, KIND = "elu", "elu"

    def __init__(self, alpha: float = 1.0, name: str = ""):
        super().__init__(name)
        self.alpha = float(alpha)

    def config_items(self):
        return [("alpha", T_FLOAT, f32(self.alpha))]


@register
class LeakyReLU(_Activation):
    TYPE_NAME, KIND = "leaky_relu", "leaky_relu"

    def __init__(self, negative_slope: float = 0.01, name: str = ""):
        super().__init__(name)
        self.alpha = float(negative_slope)

    def config_items(self):
        return [("negative_slope", T_FLOAT, f32(self.alpha))]


@register
class Activation(_Activation):
    """Generic ``activation`` layer selected by name."""
    TYPE_NAME = "activation"

    def __init__(self, activation: str = "relu", name: str = ""):
        super().__init__(name)
        if activation not in raw.ACT_KINDS:
            raise ValueError(f"unknown activation {activation!r}")
        self.KIND = activation
        self.alpha = 1.0 if activation == "elu" else 0.01 if activation == "leaky_relu" else 0.0

    def config_items(self):
        return [("activation", T_STR, self.KIND)]


# ------------------------------------------------------------------------ binary ops
class _Binary(Layer):
    OP = "add"
    n_inputs = 2

    def forward(self, inputs, ctx):
        a, b = inputs
        if self.OP in ("mul", "div"):
            ctx["a"], ctx["b"] = a, b
        return raw.binary(a, b, self.OP)

    def backward(self, grad, ctx):
        if self.OP == "add":
            return [grad, grad]
        if self.OP == "sub":
            return [grad, raw.binary(torch.zeros_like(grad), grad, "sub")]
        a, b = ctx["a"], ctx["b"]
        if self.OP == "mul":
            return [raw.binary(grad, b, "mul"), raw.binary(grad, a, "mul")]
        ga = raw.binary(grad, b, "div")
        gb = raw.binary(raw.binary(torch.zeros_like(ga), raw.binary(ga, a, "mul"), "sub"), b, "div")
        return [ga, gb]


@register
class Add(_Binary):
    TYPE_NAME, OP = "add", "add"


@register
class Sub(_Binary):
    TYPE_NAME, OP = "sub", "sub"


@register
class Mul(_Binary):
    TYPE_NAME, OP = "mul", "mul"


@register
class Div(_Binary):
    TYPE_NAME, OP = "div", "div"


# ---------------------------------------------------------------------------- dropout
@register
class Dropout(Layer):
    """Inverted dropout; the mask is regenerated from a counter-based hash in backward instead of
    being stored (reference stores a bool mask: src/nn/layers_impl/dropout_layer.cpp:26-31,91)."""
    TYPE_NAME = "dropout"

    def __init__(self, dropout_rate: float = 0.5, name: str = ""):
        super().__init__(name)
        self.dropout_rate = float(dropout_rate)

    def config_items(self):
        return [("dropout_rate", T_FLOAT, f32(self.dropout_rate))]

    def forward(self, inputs, ctx):
        p = self.dropout_rate if self.training else 0.0
        ctx["p"], ctx["seed"] = p, self.step_seed(ctx)
        return raw.dropout(inputs[0], p, ctx["seed"])

    def backward(self, grad, ctx):
        return [raw.dropout(grad, ctx["p"], ctx["seed"])]


# ------------------------------------------------------------------------- shape ops
@register
class Flatten(Layer):
    TYPE_NAME = "flatten"

    def __init__(self, start_dim: int = 1, end_dim: int = -1, name: str = ""):
        super().__init__(name)
        self.start_dim, self.end_dim = int(start_dim), int(end_dim)

    def config_items(self):
        return [("start_dim", T_INT, self.start_dim), ("end_dim", T_INT, self.end_dim)]

    def output_shape(self, in_shapes):
        s = list(in_shapes[0])
        start = max(1, self.start_dim)
        end = len(s) if self.end_dim < 0 else min(self.end_dim + 1, len(s))
        flat = 1
        for d in s[start:end]:
            flat *= d
        return tuple(s[:start]) + (flat,) + tuple(s[end:])

    def forward(self, inputs, ctx):
        x = inputs[0]
        ctx["shape"] = x.shape
        return x.reshape(self.output_shape([tuple(x.shape)]))

    def backward(self, grad, ctx):
        return [grad.reshape(ctx["shape"])]


@register
class Slice(Layer):
    """``x.narrow(axis, start, length)``. The reference declares this layer but its forward and
    backward throw (src/nn/layers_impl/slice_layer.cpp:49-60); here it works."""
    TYPE_NAME = "slice"

    def __init__(self, axis: int = 1, start: int = 0, length: int = 1, name: str = ""):
        super().__init__(name)
        self.axis, self.start, self.length = int(axis), int(start), int(length)

    def config_items(self):
        return [("axis", T_INT, self.axis), ("start", T_INT, self.start), ("length", T_INT, self.length)]

    def output_shape(self, in_shapes):
        s = list(in_shapes[0])
        s[self.axis] = self.length
        return tuple(s)

    def forward(self, inputs, ctx):
        ctx["shape"] = inputs[0].shape
        return inputs[0].narrow(self.axis, self.start, self.length).contiguous()

    def backward(self, grad, ctx):
        dx = torch.zeros(ctx["shape"], dtype=grad.dtype, device=grad.device)
        dx.narrow(self.axis, self.start, self.length).copy_(grad)
        return [dx]


@register
class Transpose(Layer):
    TYPE_NAME = "transpose"

    def __init__(self, dim0: int = 1, dim1: int = 2, name: str = ""):
        super().__init__(name)
        self.dim0, self.dim1 = int(dim0), int(dim1)

    def config_items(self):
        return [("dim0", T_SIZE, self.dim0), ("dim1", T_SIZE, self.dim1)]

    def output_shape(self, in_shapes):
        s = list(in_shapes[0])
        s[self.dim0], s[self.dim1] = s[self.dim1], s[self.dim0]
        return tuple(s)

    def forward(self, inputs, ctx):
        return inputs[0].transpose(self.dim0, self.dim1).contiguous()

    def backward(self, grad, ctx):
        return [grad.transpose(self.dim0, self.dim1).contiguous()]


# ------------------------------------------------------------------------ embeddings
@register
class Embedding(Layer):
    """Row gather; out-of-range ids read row 0, ``padding_idx`` rows are zero and get no gradient
    (src/nn/engines/cudnn_engine.cu:1196-1233). Ids are integer tensors (the reference passes them as
    floats in io_dtype, which cannot represent 50257 ids in bf16)."""
    TYPE_NAME = "embedding"

    def __init__(self, vocab_size: int, embed_dim: int, padding_idx: Optional[int] = None, name: str = ""):
        super().__init__(name)
        self.vocab_size, self.embed_dim = int(vocab_size), int(embed_dim)
        self.padding_idx = int(vocab_size if padding_idx is None else padding_idx)

    def config_items(self):
        return [("vocab_size", T_SIZE, self.vocab_size), ("embed_dim", T_SIZE, self.embed_dim),
                ("padding_idx", T_SIZE, self.padding_idx)]

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.embed_dim), True, ("normal", 1.0 / math.sqrt(self.embed_dim)))]

    def output_shape(self, in_shapes):
        return tuple(in_shapes[0]) + (self.embed_dim,)

    def forward(self, inputs, ctx):
        ids = inputs[0]
        ctx["ids"] = ids
        out = raw.embedding_fwd(ids, self.params[0], None, 1, self.padding_idx, 0.0, 0)
        return out.reshape(*ids.shape, self.embed_dim)

    def backward(self, grad, ctx):
        if self.grads[0] is not None:
            raw.embedding_bwd(ctx["ids"], _flat2d(grad), self.grads[0], None, 1, self.padding_idx, 0.0, 0)
        return [None]


@register
class PositionalEmbedding(Layer):
    """Learned ``[seq_len, E]`` table added to ``[B, S, E]``; S must equal seq_len
    (src/nn/layers_impl/positional_embedding_layer.cpp:49-53)."""
    TYPE_NAME = "pos_embedding"

    def __init__(self, embed_dim: int, seq_len: int, name: str = ""):
        super().__init__(name)
        self.embed_dim, self.seq_len = int(embed_dim), int(seq_len)

    def config_items(self):
        return [("embed_dim", T_SIZE, self.embed_dim), ("seq_len", T_SIZE, self.seq_len)]

    def param_specs(self):
        return [ParamSpec("pos", (self.seq_len, self.embed_dim), True, ("normal", 1.0 / math.sqrt(self.embed_dim)))]

    def forward(self, inputs, ctx):
        x = inputs[0]
        if x.shape[-2] != self.seq_len:
            raise ValueError(f"pos_embedding {self.name}: sequence length {x.shape[-2]} != {self.seq_len}")
        pos = self.params[0].to(x.dtype).expand_as(x).contiguous()
        return raw.binary(x.contiguous(), pos, "add")

    def backward(self, grad, ctx):
        if self.grads[0] is not None:
            raw.colsum_accum(grad.reshape(-1, self.seq_len * self.embed_dim), self.grads[0].reshape(-1))
        return [grad]


@register
class ClassToken(Layer):
    """Prepends a learned ``[E]`` token: ``[B, S, E] -> [B, S+1, E]``."""
    TYPE_NAME = "class_token"

    def __init__(self, embed_dim: int, name: str = ""):
        super().__init__(name)
        self.embed_dim = int(embed_dim)

    def config_items(self):
        return [("embed_dim", T_SIZE, self.embed_dim)]

    def param_specs(self):
        return [ParamSpec("token", (self.embed_dim,), True, ("normal", 1.0 / math.sqrt(self.embed_dim)))]

    def output_shape(self, in_shapes):
        b, s, e = in_shapes[0]
        return (b, s + 1, e)

    def forward(self, inputs, ctx):
        x = inputs[0]
        tok = self.params[0].to(x.dtype).reshape(1, 1, -1).expand(x.shape[0], 1, -1)
        return torch.cat([tok, x], 1)

    def backward(self, grad, ctx):
        if self.grads[0] is not None:
            self.grads[0].add_(grad[:, 0, :].float().sum(0))
        return [grad[:, 1:, :].contiguous()]


# ------------------------------------------------------------------------- layernorm
@register
class LayerNorm(Layer):
    TYPE_NAME = "layer_norm"

    def __init__(self, normalized_shape: int, epsilon: float = 1e-5, affine: bool = True, name: str = ""):
        super().__init__(name)
        self.normalized_shape, self.epsilon, self.affine = int(normalized_shape), float(epsilon), bool(affine)

    def config_items(self):
        return [("normalized_shape", T_SIZE, self.normalized_shape), ("epsilon", T_FLOAT, f32(self.epsilon)),
                ("affine", T_BOOL, self.affine)]

    def param_specs(self):
        if not self.affine:
            return []
        return [ParamSpec("gamma", (self.normalized_shape,), True, ("ones", 0)),
                ParamSpec("beta", (self.normalized_shape,), True, ("zeros", 0))]

    def forward(self, inputs, ctx):
        x = inputs[0]
        x2 = _flat2d(x).contiguous()
        g, b = (self.params[0], self.params[1]) if self.affine else (None, None)
        _, h, mean, rstd = raw.layernorm_fwd(x2, None, g, b, self.epsilon)
        ctx["x"], ctx["mean"], ctx["rstd"], ctx["shape"] = x2, mean, rstd, x.shape
        return h.reshape(x.shape)

    def backward(self, grad, ctx):
        g = self.params[0] if self.affine else None
        dg, db = (self.grads[0], self.grads[1]) if self.affine and self.grads[0] is not None else (None, None)
        dx, _ = raw.layernorm_bwd(_flat2d(grad), ctx["x"], ctx["mean"], ctx["rstd"], g, None, False, 0.0, 0, dg, db)
        return [dx.reshape(ctx["shape"])]


# ------------------------------------------------------------------------------- conv
@register
class Conv2D(Layer):
    """NHWC convolution with ``[O, KH, KW, I]`` weights, zero padding, no dilation/groups
    (src/nn/engines/cpu_engine.cpp:617-647)."""
    TYPE_NAME = "conv2d"

    def __init__(self, in_channels: int, out_channels: int, kernel_h: int, kernel_w: int, stride_h: int = 1,
                 stride_w: int = 1, pad_h: int = 0, pad_w: int = 0, use_bias: bool = True, name: str = ""):
        super().__init__(name)
        self.in_channels, self.out_channels = int(in_channels), int(out_channels)
        self.kernel_h, self.kernel_w = int(kernel_h), int(kernel_w)
        self.stride_h, self.stride_w, self.pad_h, self.pad_w = int(stride_h), int(stride_w), int(pad_h), int(pad_w)
        self.use_bias = bool(use_bias)

    def config_items(self):
        return [(k, T_SIZE, getattr(self, k)) for k in ("in_channels", "out_channels", "kernel_h", "kernel_w", "stride_h",
                                                        "stride_w", "pad_h", "pad_w")] + [("use_bias", T_BOOL, self.use_bias)]

    def param_specs(self):
        fan_in = self.in_channels * self.kernel_h * self.kernel_w
        std = 1.0 / math.sqrt(fan_in)
        specs = [ParamSpec("weight", (self.out_channels, self.kernel_h, self.kernel_w, self.in_channels), True, ("normal", std))]
        if self.use_bias:
            specs.append(ParamSpec("bias", (self.out_channels,), True, ("normal", std)))
        return specs

    def output_shape(self, in_shapes):
        n, h, w, _ = in_shapes[0]
        oh = (h + 2 * self.pad_h - self.kernel_h) // self.stride_h + 1
        ow = (w + 2 * self.pad_w - self.kernel_w) // self.stride_w + 1
        return (n, oh, ow, self.out_channels)

    def forward(self, inputs, ctx):
        x = inputs[0].contiguous()
        ctx["x"] = x
        # in training the patch matrix of the forward pass is kept for the weight gradient
        keep = ctx if (self.training and self.grads[0] is not None) else None
        return raw.conv2d_fwd(x, self.params[0], self.params[1] if self.use_bias else None,
                              (self.stride_h, self.stride_w), (self.pad_h, self.pad_w), keep=keep)

    def backward(self, grad, ctx):
        x = ctx["x"]
        grad = grad.contiguous()
        if self.grads[0] is not None:
            raw.conv2d_wgrad(x, grad, self.grads[0], (self.stride_h, self.stride_w), (self.pad_h, self.pad_w),
                             cols=ctx.pop("cols", None))
            if self.use_bias:
                raw.colsum_accum(_flat2d(grad), self.grads[1])
        if ctx.get("_skip_dgrad"):
            return [None]
        # "_add_to_dx": a residual block hands over the gradient of its shortcut branch; it is added here
        dx = raw.conv2d_dgrad(grad, self.params[0], x.shape, (self.stride_h, self.stride_w), (self.pad_h, self.pad_w),
                              add=ctx.pop("_add_to_dx", None))
        return [dx]


@register
class LegacyConv2D(Conv2D):
    TYPE_NAME = "legacy_conv2d"


# -------------------------------------------------------------------------- batchnorm
@register
class BatchNorm(Layer):
    """Per-channel batch norm over N*H*W with optional fused ReLU. Training normalises with the
    biased variance and updates running stats with the unbiased one; running stats are listed as
    (non-trainable) parameters so checkpoints keep the reference's 4-tensor layout
    (include/nn/layers_impl/batchnorm_layer.hpp:51-81, src/nn/engines/cpu_engine.cpp:378-511)."""
    TYPE_NAME = "batchnorm"

    def __init__(self, num_features: int, epsilon: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 use_relu: bool = False, name: str = ""):
        super().__init__(name)
        self.num_features, self.epsilon, self.momentum = int(num_features), float(epsilon), float(momentum)
        self.affine, self.use_relu = bool(affine), bool(use_relu)

    def config_items(self):
        return [("num_features", T_SIZE, self.num_features), ("epsilon", T_FLOAT, f32(self.epsilon)),
                ("momentum", T_FLOAT, f32(self.momentum)), ("affine", T_BOOL, self.affine), ("use_relu", T_BOOL, self.use_relu)]

    def param_specs(self):
        # Always four tensors, like the reference's param_descriptors: with affine = false, gamma = 1 and beta = 0
        # are still saved and loaded (files are interchangeable in both directions) but never trained or read.
        c = (self.num_features,)
        return [ParamSpec("gamma", c, self.affine, ("ones", 0)), ParamSpec("beta", c, self.affine, ("zeros", 0)),
                ParamSpec("running_mean", c, False, ("zeros", 0)), ParamSpec("running_var", c, False, ("ones", 0))]

    def _split(self):
        # gamma / beta in the compute dtype, running statistics always from the fp32 master views
        stats = getattr(self, "masters", None) or self.params
        if self.affine:
            return self.params[0], self.params[1], stats[2], stats[3]
        return None, None, stats[2], stats[3]

    def forward(self, inputs, ctx):
        x = inputs[0].contiguous()
        g, b, rm, rv = self._split()
        # A residual block whose main path ends in this layer hands over its shortcut value: the block's closing
        # add + ReLU then happens in this layer's normalisation pass (one read of the shortcut instead of a separate
        # three-tensor kernel). The ReLU belongs to the block, whose backward masks the gradient before it gets here.
        res = ctx.pop("_add_relu", None)
        # "_post_add": the graph executor hands over the other operand of the add that consumes this layer's output
        # (y = relu?(bn(x)) + other): same pass, and the backward is unchanged because the mask depends on bn(x) only
        post = ctx.pop("_post_add", None)
        relu = self.use_relu or res is not None
        if post is not None:
            res = post
        if self.training:
            y, mean, rstd = raw.batchnorm_fwd_train(x, g, b, rm, rv, self.epsilon, self.momentum, relu, resid=res,
                                                    post_add=post is not None)
            # the saved output is only read as a ReLU mask, and only where the kernels cannot recompute the mask from
            # x (no beta, or the CPU path): the executor does not hand over "_post_add" in those cases
            y_mask = y if (self.use_relu and post is None) else None
            ctx["x"], ctx["y"], ctx["mean"], ctx["rstd"] = x, y_mask, mean, rstd
            return y
        return raw.batchnorm_infer(x, g, b, rm, rv, self.epsilon, relu, resid=res, post_add=post is not None)

    def backward(self, grad, ctx):
        g, b, _, _ = self._split()
        dg, db = (self.grads[0], self.grads[1]) if self.affine and self.grads[0] is not None else (None, None)
        dx = raw.batchnorm_bwd(grad.contiguous(), ctx["x"], ctx["y"], ctx["mean"], ctx["rstd"], g, dg, db, self.use_relu, beta=b)
        return [dx]


@register
class LegacyBatchNorm(BatchNorm):
    TYPE_NAME = "legacy_batchnorm"


# ------------------------------------------------------------------------------ pools
class _Pool(Layer):
    MODE = "max"

    def __init__(self, pool_h: int, pool_w: int, stride_h: int = 0, stride_w: int = 0, pad_h: int = 0, pad_w: int = 0,
                 name: str = ""):
        super().__init__(name)
        self.pool_h, self.pool_w = int(pool_h), int(pool_w)
        self.stride_h, self.stride_w = int(stride_h) or int(pool_h), int(stride_w) or int(pool_w)
        self.pad_h, self.pad_w = int(pad_h), int(pad_w)

    def config_items(self):
        return [(k, T_SIZE, getattr(self, k)) for k in ("pool_h", "pool_w", "stride_h", "stride_w", "pad_h", "pad_w")]

    def output_shape(self, in_shapes):
        n, h, w, c = in_shapes[0]
        return (n, (h + 2 * self.pad_h - self.pool_h) // self.stride_h + 1,
                (w + 2 * self.pad_w - self.pool_w) // self.stride_w + 1, c)

    def forward(self, inputs, ctx):
        x = inputs[0].contiguous()
        y, idx = raw.pool2d_fwd(x, self.MODE, (self.pool_h, self.pool_w), (self.stride_h, self.stride_w),
                                (self.pad_h, self.pad_w), self.training)
        ctx["idx"], ctx["shape"] = idx, x.shape
        return y

    def backward(self, grad, ctx):
        return [raw.pool2d_bwd(grad.contiguous(), ctx["idx"], ctx["shape"], self.MODE, (self.pool_h, self.pool_w),
                               (self.stride_h, self.stride_w), (self.pad_h, self.pad_w))]


@register
class MaxPool2D(_Pool):
    """Window clipped to the image (padding never wins), window-relative argmax index saved
    (src/nn/engines/cpu_engine.cpp:129-210)."""
    TYPE_NAME, MODE = "maxpool2d", "max"


@register
class AvgPool2D(_Pool):
    """Divides by the number of in-image elements (src/nn/engines/cuda_engine.cu:141-194)."""
    TYPE_NAME, MODE = "avgpool2d", "avg"


@register
class LegacyMaxPool2D(MaxPool2D):
    TYPE_NAME = "legacy_maxpool2d"


@register
class LegacyAvgPool2D(AvgPool2D):
    TYPE_NAME = "legacy_avgpool2d"


# ------------------------------------------------------------------------------- sdpa
@register
class SDPA(Layer):
    """Scaled dot-product attention over three inputs q, k, v of shape ``[B, H, S, D]``."""
    TYPE_NAME = "sdpa"
    n_inputs = 3

    def __init__(self, attn_scale: float = 1.0, is_causal: bool = False, name: str = ""):
        super().__init__(name)
        self.attn_scale, self.is_causal = float(attn_scale), bool(is_causal)

    def config_items(self):
        return [("attn_scale", T_FLOAT, f32(self.attn_scale)), ("is_causal", T_BOOL, self.is_causal)]

    def forward(self, inputs, ctx):
        q, k, v = inputs
        B, H, S, D = q.shape
        packed = torch.stack([t.permute(0, 2, 1, 3).reshape(B * S, H * D) for t in (q, k, v)], 1).reshape(B * S, 3 * H * D)
        out, lse = raw.attn_fwd(packed, B, S, H, D, self.is_causal, self.attn_scale)
        ctx.update(qkv=packed, out=out, lse=lse, dims=(B, S, H, D))
        return out.reshape(B, S, H, D).permute(0, 2, 1, 3).contiguous()

    def backward(self, grad, ctx):
        B, S, H, D = ctx["dims"]
        dout = grad.permute(0, 2, 1, 3).reshape(B * S, H * D).contiguous()
        d = raw.attn_bwd(ctx["qkv"], ctx["out"], dout, ctx["lse"], B, S, H, D, self.is_causal, self.attn_scale)
        return [t.reshape(B, S, H, D).permute(0, 2, 1, 3).contiguous() for t in d.reshape(B * S, 3, H * D).unbind(1)]
