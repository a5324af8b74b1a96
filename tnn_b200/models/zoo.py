"""Model zoo: the same registry names and architectures as the reference's ``ExampleGraphs``
(src/nn/example_graphs.cpp:223-654), expressed with the :class:`~tnn_b200.nn.graph.Graph`
builder. Images are NHWC; every graph has one input node ``"input"`` and one output node
``"output"``.

Architectural facts kept from the reference: ResNet-50 uses a biased 7x7/2 stem, BN+ReLU after
every conv of a bottleneck *including the last one* and no ReLU after the residual add
(``:176-196``); WRN-16-8 blocks are pre-activation with biased convs and dropout 0.3
(``:153-174``); GPT-2 is pre-LN with learned positions, dropout 0.1, tanh-GELU and an untied,
biased vocabulary head (``:198-215,588-611``).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple

from ..nn.blocks import FlashAttentionBlock
from ..nn.graph import Graph, Node
from ..nn.layers import (AvgPool2D, BatchNorm, ClassToken, Conv2D, Dense, Dropout, Embedding, Flatten, GELU, LayerNorm,
                         MaxPool2D, PositionalEmbedding, ReLU, Slice)

BN_EPS = 1e-5
BN_MOMENTUM = 0.1


class _B:
    """Tracks the running activation shape while layers are appended (shape excludes nothing: NHWC)."""

    def __init__(self, graph: Graph, node: Node, shape: Tuple[int, ...]):
        self.g, self.x, self.shape = graph, node, tuple(shape)

    def fork(self) -> "_B":
        return _B(self.g, self.x, self.shape)

    def apply(self, layer) -> "_B":
        self.shape = layer.output_shape([self.shape])
        self.x = layer(self.x)
        return self

    def conv(self, out_c, k, stride=1, pad=0, bias=False, name=""):
        return self.apply(Conv2D(self.shape[-1], out_c, k, k, stride, stride, pad, pad, bias, name=name))

    def bn(self, relu, name=""):
        return self.apply(BatchNorm(self.shape[-1], BN_EPS, BN_MOMENTUM, True, relu, name=name))

    def maxpool(self, k, s, p=0, name=""):
        return self.apply(MaxPool2D(k, k, s, s, p, p, name=name))

    def avgpool(self, k, s=1, p=0, name=""):
        return self.apply(AvgPool2D(k, k, s, s, p, p, name=name))

    def flatten(self, start=1, end=-1, name="flatten"):
        return self.apply(Flatten(start, end, name=name))

    def dense(self, out_f, bias=True, name=""):
        return self.apply(Dense(self.shape[-1], out_f, bias, name=name))

    def relu(self, name=""):
        return self.apply(ReLU(name=name))

    def dropout(self, p, name=""):
        return self.apply(Dropout(p, name=name))

    def layernorm(self, eps=1e-5, name=""):
        return self.apply(LayerNorm(self.shape[-1], eps, True, name=name))

    def add(self, other: "_B") -> "_B":
        self.x = self.x + other.x
        return self


def _start(shape) -> _B:
    g = Graph()
    return _B(g, g.input("input"), shape)


def _finish(b: _B) -> Graph:
    b.x.set_uid("output")
    b.g.set_output(b.x)
    return b.g


# ---------------------------------------------------------------------- residual blocks
def basic_block(b: _B, out_c: int, stride: int, name: str) -> _B:
    main = b.fork().conv(out_c, 3, stride, 1, False, name + "_conv1").bn(True, name + "_bn0")
    main.conv(out_c, 3, 1, 1, False, name + "_conv2").bn(False, name + "_bn1")
    sc = b.fork()
    if stride != 1 or b.shape[-1] != out_c:
        sc.conv(out_c, 1, stride, 0, False, name + "_conv0").bn(False, name + "_shortcut_bn")
    main.add(sc)
    return main.relu(name + "_relu")


def wide_block(b: _B, out_c: int, stride: int, drop: float, name: str) -> _B:
    main = b.fork().bn(True, name + "_bn1").conv(out_c, 3, stride, 1, True, name + "_conv1").bn(True, name + "_bn2")
    if drop > 0:
        main.dropout(drop, name + "_dropout")
    main.conv(out_c, 3, 1, 1, True, name + "_conv2")
    sc = b.fork()
    if stride != 1 or b.shape[-1] != out_c:
        sc.conv(out_c, 1, stride, 0, False, name + "_shortcut_conv")
    return main.add(sc)


def bottleneck_block(b: _B, mid_c: int, out_c: int, stride: int, name: str) -> _B:
    main = b.fork().conv(mid_c, 1, 1, 0, False, name + "_conv1").bn(True, name + "_bn0")
    main.conv(mid_c, 3, stride, 1, False, name + "_conv2").bn(True, name + "_bn1")
    main.conv(out_c, 1, 1, 0, False, name + "_conv3").bn(True, name + "_bn2")
    sc = b.fork()
    if stride != 1 or b.shape[-1] != out_c:
        sc.conv(out_c, 1, stride, 0, False, name + "_conv0").bn(False, name + "_bn3")
    return main.add(sc)


def gpt_block(b: _B, embed: int, heads: int, ffn: int, drop: float, causal: bool, name: str) -> _B:
    attn = b.fork().layernorm(1e-5, name + "_ln_1")
    attn.apply(FlashAttentionBlock(embed, heads, causal, name=name + "_attn")).dropout(drop, name + "_attn_dropout")
    x = b.fork().add(attn)
    ffn_b = x.fork().layernorm(1e-5, name + "_ln_2").dense(ffn, True, name + "_mlp_fc1")
    ffn_b.apply(GELU(name=name + "_mlp_activation")).dense(embed, True, name + "_mlp_fc2").dropout(drop, name + "_mlp_dropout")
    return x.add(ffn_b)


# ------------------------------------------------------------------------------ models
def mnist_cnn() -> Graph:
    b = _start((1, 28, 28, 1))
    b.conv(8, 5, 1, 0, False, "conv1").bn(True, "bn1").maxpool(3, 3, 0, "pool1")
    b.conv(16, 1, 1, 0, False, "conv2_1x1").bn(True, "bn2_1x1").relu("relu2")
    b.conv(48, 5, 1, 0, False, "conv3").bn(True, "bn3").maxpool(2, 2, 0, "pool2")
    return _finish(b.flatten().dense(10, False, "output"))


def cifar10_vgg() -> Graph:
    b = _start((1, 32, 32, 3))
    plan = [(64, "0", True), (64, "1", True), "pool0", (128, "2", True), (128, "3", True), "pool1", (256, "4", True),
            (256, "5", False), (256, "6", True), "pool2", (512, "7", True), (512, "8", True), (512, "9", True), "pool3"]
    for item in plan:
        if isinstance(item, str):
            b.maxpool(2, 2, 0, item)
        else:
            c, tag, with_bn = item
            b.conv(c, 3, 1, 1, False, "conv" + tag)
            if with_bn:
                b.bn(True, "bn" + tag)
            else:
                b.relu("relu" + tag)
    b.flatten().dense(512, True, "fc0").relu("relu10")
    return _finish(b.dense(10, True, "fc1"))


def cifar10_test() -> Graph:
    b = _start((1, 32, 32, 3))
    b.conv(64, 3, 1, 1, False, "conv1").bn(True, "bn1").conv(128, 3, 1, 1, False, "conv2").bn(True, "bn2").maxpool(2, 2, 0, "pool1")
    b = basic_block(b, 256, 1, "res_block1").maxpool(2, 2, 0, "pool2")
    b = basic_block(b, 512, 1, "res_block2").maxpool(2, 2, 0, "pool3")
    return _finish(b.avgpool(4, 1, 0, "avgpool").flatten().dense(10, True, "output"))


def cifar10_resnet9() -> Graph:
    b = _start((1, 32, 32, 3))
    b.conv(64, 3, 1, 1, False, "conv1").bn(True, "bn1").conv(128, 3, 1, 1, False, "conv2").bn(True, "bn2").maxpool(2, 2, 0, "pool1")
    b = basic_block(basic_block(b, 128, 1, "res_block1"), 128, 1, "res_block2")
    b.conv(256, 3, 1, 1, False, "conv3").bn(True, "bn3").maxpool(2, 2, 0, "pool2")
    b = basic_block(basic_block(b, 256, 1, "res_block3"), 256, 1, "res_block4")
    b.conv(512, 3, 1, 1, False, "conv4").bn(True, "bn4").maxpool(2, 2, 0, "pool3")
    b = basic_block(b, 512, 1, "res_block5")
    return _finish(b.avgpool(4, 1, 0, "avgpool").flatten().dense(10, True, "output"))


def _resnet18(side: int, classes: int, pool: int) -> Graph:
    b = _start((1, side, side, 3))
    b.conv(32, 3, 1, 1, False, "conv1").bn(True, "bn1").maxpool(2, 2, 0, "maxpool")
    for li, (c, s) in enumerate([(64, 1), (128, 2), (256, 2), (512, 2)], 1):
        b = basic_block(b, c, s, f"layer{li}_block1")
        b = basic_block(b, c, 1, f"layer{li}_block2")
    return _finish(b.avgpool(pool, 1, 0, "avgpool").flatten().dense(classes, True, "fc"))


def _wrn16_8(side: int, classes: int) -> Graph:
    b = _start((1, side, side, 3))
    b.conv(16, 3, 1, 1, True, "conv1")
    for gi, (c, s) in enumerate([(128, 1), (256, 2), (512, 2)], 1):
        b = wide_block(b, c, s, 0.3, f"group{gi}_block1")
        b = wide_block(b, c, 1, 0.3, f"group{gi}_block2")
    b.bn(True, "bn_final")
    return _finish(b.avgpool(8, 1, 0, "avgpool").flatten().dense(classes, True, "fc"))


def _resnet50(side: int, classes: int, imagenet_stem: bool, pool: int) -> Graph:
    b = _start((1, side, side, 3))
    if imagenet_stem:
        b.conv(64, 7, 2, 3, True, "conv1")
    else:
        b.conv(64, 3, 1, 1, True, "conv1")
    b.bn(True, "bn1").maxpool(3, 2, 1, "maxpool")
    for li, (mid, out, n, s) in enumerate([(64, 256, 3, 1), (128, 512, 4, 2), (256, 1024, 6, 2), (512, 2048, 3, 2)], 1):
        for bi in range(n):
            b = bottleneck_block(b, mid, out, s if bi == 0 else 1, f"layer{li}_block{bi + 1}")
    return _finish(b.avgpool(pool, 1, 0, "avgpool").flatten().dense(classes, True, "fc"))


def _vit() -> Graph:
    patch, embed, heads, depth, classes = 4, 256, 4, 4, 200
    seq = (64 // patch) ** 2 + 1
    b = _start((1, 64, 64, 3))
    b.conv(embed, patch, patch, 0, True, "patch_embed").flatten(1, 2, "flatten_patches")
    b.apply(ClassToken(embed, name="class_token")).apply(PositionalEmbedding(embed, seq, name="positional_embedding"))
    b.dropout(0.1, "dropout")
    for i in range(depth):
        b = gpt_block(b, embed, heads, embed * 4, 0.1, False, f"encoder_{i}")
    b.layernorm(1e-5, "ln_final").apply(Slice(1, 0, 1, name="extract_cls")).flatten(1, -1, "flatten_cls")
    return _finish(b.dense(classes, True, "head"))


def gpt2(embed: int, heads: int, layers: int, name: str, seq_len: int = 1024, vocab: int = 50257, drop: float = 0.1) -> Graph:
    b = _start((1, seq_len))
    b.apply(Embedding(vocab, embed, name="token_embed")).apply(PositionalEmbedding(embed, seq_len, name="pos_embed"))
    b.dropout(drop, "dropout")
    for i in range(layers):
        b = gpt_block(b, embed, heads, embed * 4, drop, True, f"{name}_block_{i}")
    b.layernorm(1e-5, "ln_f")
    return _finish(b.dense(vocab, True, "head"))


MODEL_REGISTRY: Dict[str, Callable[[], Graph]] = {
    "mnist_cnn": mnist_cnn,
    "cifar10_vgg": cifar10_vgg,
    "cifar10_test": cifar10_test,
    "cifar10_resnet9": cifar10_resnet9,
    "cifar100_resnet18": lambda: _resnet18(32, 100, 2),
    "cifar100_wrn16_8": lambda: _wrn16_8(32, 100),
    "tiny_imagenet_resnet18": lambda: _resnet18(64, 200, 4),
    "tiny_imagenet_wrn16_8": lambda: _wrn16_8(64, 200),
    "tiny_imagenet_resnet50": lambda: _resnet50(64, 200, False, 4),
    "tiny_imagenet_vit": _vit,
    "tiny_imagenet_flash_vit": _vit,
    "imagenet_resnet50": lambda: _resnet50(224, 1000, True, 7),
    "imagenet100_resnet50": lambda: _resnet50(224, 100, True, 7),
    "gpt2_small": lambda: gpt2(768, 12, 12, "gpt2_small"),
    "flash_gpt2_small": lambda: gpt2(768, 12, 12, "flash_gpt2_small"),
    "gpt2_medium": lambda: gpt2(1024, 16, 24, "gpt2_medium"),
    "flash_gpt2_medium": lambda: gpt2(1024, 16, 24, "flash_gpt2_medium"),
    "gpt2_large": lambda: gpt2(1280, 20, 36, "gpt2_large"),
    "flash_gpt2_large": lambda: gpt2(1280, 20, 36, "flash_gpt2_large"),
}

INPUT_SHAPES: Dict[str, Tuple[int, ...]] = {
    "mnist_cnn": (28, 28, 1), "cifar10_vgg": (32, 32, 3), "cifar10_test": (32, 32, 3), "cifar10_resnet9": (32, 32, 3),
    "cifar100_resnet18": (32, 32, 3), "cifar100_wrn16_8": (32, 32, 3), "tiny_imagenet_resnet18": (64, 64, 3),
    "tiny_imagenet_wrn16_8": (64, 64, 3), "tiny_imagenet_resnet50": (64, 64, 3), "tiny_imagenet_vit": (64, 64, 3),
    "tiny_imagenet_flash_vit": (64, 64, 3), "imagenet_resnet50": (224, 224, 3), "imagenet100_resnet50": (224, 224, 3),
}


def register_model(name: str, builder: Callable[[], Graph]) -> None:
    MODEL_REGISTRY[name] = builder


def available_models() -> List[str]:
    return sorted(MODEL_REGISTRY)


def create(name: str, **compile_kw) -> Graph:
    """Build a zoo model; with keyword arguments the graph is also compiled (``device=...``)."""
    if name not in MODEL_REGISTRY:
        raise KeyError(f"unknown model {name!r}; available: {available_models()}")
    g = MODEL_REGISTRY[name]()
    if compile_kw:
        g.compile(**compile_kw)
    return g
