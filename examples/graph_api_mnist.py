"""A small CNN assembled with the graph-builder API and trained for a few steps on synthetic MNIST-shaped data.

conv3x3(32) - relu - maxpool - conv3x3(64) - relu - maxpool - flatten - dense(128) - relu - dense(10), with a
skip connection added around the second convolution to show ``node + node``.
Reference: examples/graph_api_v2_test.cpp:13-100.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.nn import layers as L  # noqa: E402
from tnn_b200.nn.graph import Graph  # noqa: E402
from tnn_b200.nn.loss import CrossEntropyLoss  # noqa: E402
from tnn_b200.nn.optim import SGD  # noqa: E402


def build() -> Graph:
    g = Graph()
    x = g.input("input")
    h = L.Conv2D(1, 32, 3, 3, 1, 1, 1, 1, name="conv1")(x)
    h = L.Activation("relu", name="relu1")(h)
    h = L.MaxPool2D(2, 2, 2, 2, name="pool1")(h)
    c2 = L.Conv2D(32, 32, 3, 3, 1, 1, 1, 1, name="conv2")(h)
    h = L.Activation("relu", name="relu2")(c2 + h)  # residual connection through the graph's add
    h = L.Conv2D(32, 64, 3, 3, 1, 1, 1, 1, name="conv3")(h)
    h = L.Activation("relu", name="relu3")(h)
    h = L.MaxPool2D(2, 2, 2, 2, name="pool2")(h)
    h = L.Flatten(name="flatten")(h)
    h = L.Dense(7 * 7 * 64, 128, name="fc1")(h)
    h = L.Activation("relu", name="relu4")(h)
    out = L.Dense(128, 10, name="fc2")(h)
    out.set_uid("output")
    g.set_output(out)
    return g


def main(steps: int = 40, batch: int = 32, device: str = "cpu"):
    g = build().compile(device=device, seed=0)
    opt = SGD(learning_rate=0.01, momentum=0.9).attach(g)
    loss_fn = CrossEntropyLoss()
    gen = torch.Generator().manual_seed(0)
    protos = torch.randn(10, 28, 28, 1, generator=gen)  # one prototype image per class + noise
    first = last = None
    for step in range(steps):
        labels = torch.randint(0, 10, (batch,), generator=gen)
        data = protos[labels] + 0.3 * torch.randn(batch, 28, 28, 1, generator=gen)
        if device != "cpu":
            data, labels = data.to(device).to(g.io_dtype), labels.to(device)
        out = g.forward({"input": data})["output"]
        loss, grad = loss_fn.compute(out, labels)
        g.backward({"output": grad})
        opt.update()
        g.zero_grads()
        last = float(loss)
        first = last if first is None else first
        if step % 10 == 0:
            print(f"step {step} loss {last:.4f}")
    print(f"loss {first:.4f} -> {last:.4f}")
    return first, last


if __name__ == "__main__":
    main(device="cuda" if torch.cuda.is_available() else "cpu")
