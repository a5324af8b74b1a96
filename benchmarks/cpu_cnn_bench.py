#!/usr/bin/env python
"""CPU, fp32, single process: the small CNN benchmark configuration.

    python benchmarks/cpu_cnn_bench.py [--steps 100] [--batch 64] [--threads N]

Synthetic 28x28x1 images (pixels uniform in [0,1)), labels uniform in [0,10), batch 64; conv3x3(32)+ReLU,
maxpool2, conv3x3(64)+ReLU, maxpool2, dense 128+ReLU, dense 10, softmax cross-entropy; SGD lr 0.01, seed 0,
100 steps. The network is not a zoo model, so it is assembled with the public graph-builder API, as the
reference's examples/graph_api_v2_test.cpp:13-80 does.

Two arms run the same steps from the same initial weights on the same data:

* ``framework``: the graph executor on ``device="cpu"`` (the layers' CPU path, vectorised tensor ops);
* ``cpu_engine``: the C++ fp32 NHWC engine (``host.H.cpu``), which restates the arithmetic of the reference's
  CPU engine - direct 7-loop convolutions (src/nn/engines/cpu_engine.cpp:617-734), sgemm dense (:25-44),
  clipped-window max-pool (:129-210) - and is the timed CPU baseline and the numerical oracle.

One JSON line per arm (``steps_per_sec``, ``images_per_sec``, first / last loss) and one line comparing the
loss curves of the two arms.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.host import H  # noqa: E402
from tnn_b200.nn import layers as L  # noqa: E402
from tnn_b200.nn.graph import Graph  # noqa: E402
from tnn_b200.nn.loss import CrossEntropyLoss  # noqa: E402
from tnn_b200.nn.optim import SGD  # noqa: E402


def build() -> Graph:
    g = Graph()
    h = g.input("input")
    h = L.Conv2D(1, 32, 3, 3, 1, 1, 0, 0, name="conv1")(h)
    h = L.Activation("relu", name="relu1")(h)
    h = L.MaxPool2D(2, 2, 2, 2, name="pool1")(h)          # 26 -> 13
    h = L.Conv2D(32, 64, 3, 3, 1, 1, 0, 0, name="conv2")(h)
    h = L.Activation("relu", name="relu2")(h)
    h = L.MaxPool2D(2, 2, 2, 2, name="pool2")(h)          # 11 -> 5
    h = L.Flatten(name="flatten")(h)
    h = L.Dense(5 * 5 * 64, 128, name="fc1")(h)
    h = L.Activation("relu", name="relu3")(h)
    out = L.Dense(128, 10, name="fc2")(h)
    out.set_uid("output")
    g.set_output(out)
    return g


def batches(steps: int, batch: int):
    gen = torch.Generator().manual_seed(0)
    return [(torch.rand(batch, 28, 28, 1, generator=gen), torch.randint(0, 10, (batch,), generator=gen)) for _ in range(steps)]


def run_framework(data, lr: float):
    g = build().compile(device="cpu", seed=0)
    init = [p.detach().clone() for p in g.parameters()]
    opt = SGD(learning_rate=lr, momentum=0.0).attach(g)
    loss_fn = CrossEntropyLoss()
    g.train()
    losses = []
    t0 = time.perf_counter()
    for x, y in data:
        out = g.forward({"input": x})["output"]
        loss, grad = loss_fn.compute(out, y)
        g.backward({"output": grad})
        opt.update()
        g.zero_grads()
        losses.append(float(loss))
    return time.perf_counter() - t0, losses, init


def run_cpu_engine(data, lr: float, init):
    c = H.cpu
    w1, b1, w2, b2, w3, b3, w4, b4 = [np.ascontiguousarray(p.float().numpy()).copy() for p in init]
    params = [w1, b1, w2, b2, w3, b3, w4, b4]
    grads = [np.zeros_like(p) for p in params]
    losses = []
    t0 = time.perf_counter()
    for x, y in data:
        x0 = np.ascontiguousarray(x.numpy())
        lab = np.ascontiguousarray(y.numpy().astype(np.int32))
        a1 = c.conv2d_fwd(x0, w1, b1, 1, 1, 0, 0)
        r1 = c.relu_fwd(a1)
        p1, i1 = c.pool2d_fwd(r1, True, 2, 2, 2, 2, 0, 0)
        a2 = c.conv2d_fwd(p1, w2, b2, 1, 1, 0, 0)
        r2 = c.relu_fwd(a2)
        p2, i2 = c.pool2d_fwd(r2, True, 2, 2, 2, 2, 0, 0)
        f = p2.reshape(p2.shape[0], -1)
        a3 = c.dense_fwd(f, w3, b3)
        r3 = c.relu_fwd(a3)
        a4 = c.dense_fwd(r3, w4, b4)
        loss, dz, _ = c.softmax_ce(a4, lab)
        losses.append(float(loss))
        for g_ in grads:
            g_.fill(0.0)
        d3 = c.dense_bwd(dz, r3, w4, grads[6], grads[7])
        d3 = c.relu_bwd(a3, d3)
        df = c.dense_bwd(d3, f, w3, grads[4], grads[5])
        dp2 = c.pool2d_bwd(np.ascontiguousarray(df.reshape(p2.shape)), i2, list(r2.shape), True, 2, 2, 2, 2, 0, 0)
        da2 = c.relu_bwd(a2, dp2)
        c.conv2d_wgrad(p1, da2, grads[2], grads[3], 1, 1, 0, 0)
        dp1 = c.conv2d_dgrad(da2, w2, list(p1.shape), 1, 1, 0, 0)
        dr1 = c.pool2d_bwd(dp1, i1, list(r1.shape), True, 2, 2, 2, 2, 0, 0)
        da1 = c.relu_bwd(a1, dr1)
        c.conv2d_wgrad(x0, da1, grads[0], grads[1], 1, 1, 0, 0)
        for p, g_ in zip(params, grads):
            c.sgd_step(p, g_, None, lr, 0.0)
    return time.perf_counter() - t0, losses


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--threads", type=int, default=0, help="torch / OpenMP threads (0 = library default)")
    args = ap.parse_args()
    if args.threads:
        torch.set_num_threads(args.threads)
    data = batches(args.steps, args.batch)
    common = {"config": "small CNN 28x28x1, fp32, CPU, single process", "batch": args.batch, "steps": args.steps, "optimizer": "sgd",
              "lr": args.lr, "seed": 0, "threads": torch.get_num_threads(), "data": "synthetic (uniform pixels, uniform labels)"}
    t_f, l_f, init = run_framework(data, args.lr)
    print(json.dumps({**common, "arm": "framework", "seconds": round(t_f, 3), "steps_per_sec": round(args.steps / t_f, 2),
                      "images_per_sec": round(args.steps * args.batch / t_f, 1), "loss_first": round(l_f[0], 4), "loss_last": round(l_f[-1], 4)}))
    t_e, l_e = run_cpu_engine(data, args.lr, init)
    print(json.dumps({**common, "arm": "cpu_engine", "seconds": round(t_e, 3), "steps_per_sec": round(args.steps / t_e, 2),
                      "images_per_sec": round(args.steps * args.batch / t_e, 1), "loss_first": round(l_e[0], 4), "loss_last": round(l_e[-1], 4)}))
    diff = max(abs(a - b) for a, b in zip(l_f, l_e))
    print(json.dumps({"max_loss_difference_between_arms": round(diff, 6), "speedup_framework_over_cpu_engine": round(t_e / t_f, 2)}))


if __name__ == "__main__":
    main()
