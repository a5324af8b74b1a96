#!/usr/bin/env python
"""Operator micro-benchmarks (the counterpart of the reference's benchmarks/*.cpp: gemm, dense,
attention block, batchnorm, conv2d ...). Each sub-command times one kernel with CUDA events after
warm-up, on inputs larger than the 126 MB L2 or with an L2 flush between iterations, and prints
achieved bandwidth / FLOP rate. Also the programs the ncu summaries under profiles/ were made with.

    python benchmarks/microbench.py gemm --m 8192 --n 3072 --k 768
    python benchmarks/microbench.py attention --batch 8 --heads 12 --seq 1024
    python benchmarks/microbench.py layernorm --rows 65536 --cols 768
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.ops import _lib, raw  # noqa: E402
from tnn_b200.ops.gemm import gemm  # noqa: E402

_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        # larger than the 126 MB L2, and long enough to write (about 0.2 ms) that the host-side work of the timed
        # call - argument checks, tensor maps, the launch itself - is over before the GPU gets to the start event
        _FLUSH = torch.empty(1024 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timeit(fn, iters, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def bf(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def cmd_gemm(a):
    M, N, K = a.m, a.n, a.k
    res = {}
    x, w = bf(M, K), bf(N, K)
    res["fwd_ms"] = timeit(lambda: gemm(x, w, force_bn=a.bn), a.iters)
    if a.all:
        dy = bf(M, N)
        dw = torch.zeros(N, K, device="cuda")
        res["dgrad_ms"] = timeit(lambda: gemm(dy, w, b_t=True), a.iters)
        res["wgrad_ms"] = timeit(lambda: gemm(dy, x, a_t=True, b_t=True, out=dw, atomic=True), a.iters)
        res["torch_fwd_ms"] = timeit(lambda: x @ w.t(), a.iters)
        # the two GELU forms of the MLP: forward with bias + GELU and a saved pre-activation, data gradient times GELU'
        bias, z, out = bf(N), torch.empty(M, N, device="cuda", dtype=torch.bfloat16), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        res["fwd_bias_gelu_ms"] = timeit(lambda: gemm(x, w, bias=bias, gelu=True, save_preact=z, out=out), a.iters)
        zk, dxo = bf(M, K), torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        res["dgrad_dgelu_ms"] = timeit(lambda: gemm(dy, w, b_t=True, dgelu_of=zk, out=dxo), a.iters)
    fl = 2.0 * M * N * K
    for k in list(res):
        res[k.replace("_ms", "_tflops")] = round(fl / res[k] / 1e9, 1)
    return res


def cmd_attention(a):
    B, S, H, D = a.batch, a.seq, a.heads, 64
    qkv = bf(B * S, 3 * H * D)
    out, lse = raw.attn_fwd(qkv, B, S, H, D, True, 0.125)
    do = bf(B * S, H * D)
    fl = 4.0 * B * H * S * S * D / 2
    f = timeit(lambda: raw.attn_fwd(qkv, B, S, H, D, True, 0.125), a.iters)
    b = timeit(lambda: raw.attn_bwd(qkv, out, do, lse, B, S, H, D, True, 0.125), a.iters)
    res = {"fwd_ms": f, "fwd_tflops": round(fl / f / 1e9, 1), "bwd_ms": b, "bwd_tflops": round(2.5 * fl / b / 1e9, 1)}
    if a.library:
        res.update(_sdpa_library(qkv, do, B, S, H, D, a.iters))
    return res


def _sdpa_library(qkv, do, B, S, H, D, iters):
    """The same attention through torch.nn.functional.scaled_dot_product_attention restricted to the cuDNN backend
    (the library call of the reference's engine, src/nn/engines/cudnn_engine.cu:1479-1621), else the flash backend."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel
    q, k, v = (t.permute(0, 2, 1, 3) for t in qkv.view(B, S, 3, H, D).unbind(2))  # [B, H, S, D] views, no copies
    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    g = do.view(B, S, H, D).permute(0, 2, 1, 3)
    for name, be in (("cudnn", SDPBackend.CUDNN_ATTENTION), ("flash", SDPBackend.FLASH_ATTENTION)):
        try:
            with sdpa_kernel([be]):
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.125)
                f = timeit(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.125), iters)
                b = timeit(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), iters)
            return {"library": "torch sdpa / " + name, "lib_fwd_ms": f, "lib_bwd_ms": b}
        except Exception as e:  # backend not available for this shape / build
            last = f"{name}: {type(e).__name__}"
    return {"library": "unavailable (" + last + ")"}


def cmd_layernorm(a):
    R, C = a.rows, a.cols
    x, d, g, b = bf(R, C), bf(R, C), bf(C) + 1, bf(C)
    f = timeit(lambda: raw.layernorm_fwd(x, d, g, b, 1e-5, 0.1, 1), a.iters)
    xo, h, mean, rstd = raw.layernorm_fwd(x, d, g, b, 1e-5, 0.1, 1)
    dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    bw = timeit(lambda: raw.layernorm_bwd(h, xo, mean, rstd, g, x, True, 0.1, 1, dg, db), a.iters)
    byt = R * C * 2
    return {"fwd_ms": f, "fwd_gbs": round(4 * byt / f / 1e6), "bwd_ms": bw, "bwd_gbs": round(5 * byt / bw / 1e6)}


def cmd_softmax_ce(a):
    R, V = a.rows, a.vocab
    ld = (V + 63) // 64 * 64
    lg = bf(R, ld, scale=2.0)
    lab = torch.randint(0, V, (R,), device="cuda")
    t = timeit(lambda: raw.softmax_ce(lg[:, :V], lab, V, 1.0 / R, 1.0 / R, grad_out=lg[:, :V]), a.iters)
    return {"ms": t, "gbs": round(2 * R * ld * 2 / t / 1e6)}


def cmd_colsum(a):
    R, C = a.rows, a.cols
    dy = bf(R, C)
    db = torch.zeros(C, device="cuda")
    t = timeit(lambda: raw.colsum_accum(dy, db), a.iters)
    return {"ms": t, "gbs": round(R * C * 2 / t / 1e6)}


def cmd_adam(a):
    n = a.n
    w, g, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    lp = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: raw.adam_step(w, lp, g, m, v, 1e-3, 0.9, 0.99, 1e-8, 0.0, 1), a.iters, flush=False)
    return {"ms": t, "gbs": round(n * 30 / t / 1e6)}


def cmd_conv2d(a):
    x = bf(a.batch, a.size, a.size, a.cin)
    w = bf(a.cout, a.ksize, a.ksize, a.cin, scale=0.05)
    st, pd = (a.stride, a.stride), (a.ksize // 2, a.ksize // 2)
    y = raw.conv2d_fwd(x, w, None, st, pd)
    dy = torch.randn_like(y)
    dw = torch.zeros(w.shape, device="cuda")
    fl = 2.0 * y.numel() * a.ksize * a.ksize * a.cin
    f = timeit(lambda: raw.conv2d_fwd(x, w, None, st, pd), a.iters)
    d = timeit(lambda: raw.conv2d_dgrad(dy, w, x.shape, st, pd), a.iters)
    g = timeit(lambda: raw.conv2d_wgrad(x, dy, dw, st, pd), a.iters)
    res = {"fwd_ms": f, "fwd_tflops": round(fl / f / 1e9, 1), "dgrad_ms": d, "dgrad_tflops": round(fl / d / 1e9, 1),
           "wgrad_ms": g, "wgrad_tflops": round(fl / g / 1e9, 1)}
    if a.library:
        try:
            res.update(_conv_library(x, w, dy, st, pd, a.iters))
        except Exception as e:  # keep this package's figures if the library path refuses the shape
            res["library_error"] = f"{type(e).__name__}: {str(e)[:120]}"
    return res


def _conv_library(x, w, dy, st, pd, iters):
    """The same three passes through cuDNN as torch dispatches them (bf16, channels-last views of the NHWC tensors,
    autotuned): the library the reference's engine builds its convolution graphs on
    (src/nn/engines/cudnn_engine.cu:328-578)."""
    torch.backends.cudnn.benchmark = True
    xt, wt, gt = x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), dy.permute(0, 3, 1, 2)
    conv = torch.ops.aten.convolution_backward
    args = (list(st), list(pd), [1, 1], False, [0, 0], 1)
    f = timeit(lambda: torch.nn.functional.conv2d(xt, wt, None, st, pd), iters)
    d = timeit(lambda: conv(gt, xt, wt, None, *args, [True, False, False]), iters)
    g = timeit(lambda: conv(gt, xt, wt, None, *args, [False, True, False]), iters)
    return {"lib_fwd_ms": f, "lib_dgrad_ms": d, "lib_wgrad_ms": g}


# every distinct convolution of ResNet-50 at 224 x 224: (input size, C, O, filter, stride)
_RESNET50_CONVS = [(224, 3, 64, 7, 2),
                   (56, 64, 64, 1, 1), (56, 64, 64, 3, 1), (56, 64, 256, 1, 1), (56, 256, 64, 1, 1),
                   (56, 256, 128, 1, 1), (56, 128, 128, 3, 2), (28, 128, 512, 1, 1), (56, 256, 512, 1, 2), (28, 512, 128, 1, 1),
                   (28, 128, 128, 3, 1),
                   (28, 512, 256, 1, 1), (28, 256, 256, 3, 2), (14, 256, 1024, 1, 1), (28, 512, 1024, 1, 2), (14, 1024, 256, 1, 1),
                   (14, 256, 256, 3, 1),
                   (14, 1024, 512, 1, 1), (14, 512, 512, 3, 2), (7, 512, 2048, 1, 1), (14, 1024, 2048, 1, 2), (7, 2048, 512, 1, 1),
                   (7, 512, 512, 3, 1)]


def cmd_conv_table(a):
    """One line per distinct ResNet-50 convolution: this package's kernels beside cuDNN (through torch)."""
    rows = []
    for size, cin, cout, k, stride in _RESNET50_CONVS:
        ns = argparse.Namespace(batch=a.batch, size=size, cin=cin, cout=cout, ksize=k, stride=stride, iters=a.iters, library=True)
        r = cmd_conv2d(ns)
        row = {"shape": f"{size}x{size}x{cin}->{cout} k{k} s{stride}", **{key: round(v, 4) for key, v in r.items()}}
        print(json.dumps(row), flush=True)
        rows.append(row)
    tot = {key: round(sum(r.get(key, 0.0) for r in rows), 3) for key in ("fwd_ms", "dgrad_ms", "wgrad_ms", "lib_fwd_ms", "lib_dgrad_ms", "lib_wgrad_ms")}
    return {"layers": len(rows), **tot}


def cmd_batchnorm(a):
    x = bf(a.batch, a.size, a.size, a.channels)
    C = a.channels
    g, b = bf(C) + 1, bf(C)
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    f = timeit(lambda: raw.batchnorm_fwd_train(x, g, b, rm, rv, 1e-5, 0.1, True), a.iters)
    y, mean, rstd = raw.batchnorm_fwd_train(x, g, b, rm, rv, 1e-5, 0.1, True)
    dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    bw = timeit(lambda: raw.batchnorm_bwd(y, x, y, mean, rstd, g, dg, db, True, beta=b), a.iters)
    byt = x.numel() * 2
    return {"fwd_ms": f, "fwd_gbs": round(3 * byt / f / 1e6), "bwd_ms": bw, "bwd_gbs": round(5 * byt / bw / 1e6)}


def _time_graph(g, x, iters):
    """Forward + backward of a compiled graph through the executor (the calls a user makes), device-timed."""
    out = g.forward({"input": x})["output"]
    dy = torch.randn_like(out)
    g.backward({"output": dy})
    f = timeit(lambda: g.forward({"input": x}), iters)

    def fb():
        g.forward({"input": x})
        g.backward({"output": dy})
        g.zero_grads()

    return f, timeit(fb, iters)


def cmd_attention_block(a):
    """The reference's attention-block benchmark (benchmarks/attention_benchmark.cpp:11-40: batch 16, sequence 512,
    embedding 768, 8 heads, i.e. head size 96): QKV projection, causal attention and output projection as one layer."""
    from tnn_b200.nn.blocks import FlashAttentionBlock
    from tnn_b200.nn.graph import Graph

    g = Graph()
    out = FlashAttentionBlock(a.embed, a.heads, True, 1.0 / (a.embed // a.heads) ** 0.5, name="attn")(g.input("input"))
    out.set_uid("output")
    g.set_output(out)
    g.input_requires_grad = True
    g.compile(device="cuda", seed=0)
    x = bf(a.batch, a.seq, a.embed)
    f, fb = _time_graph(g, x, a.iters)
    D = a.embed // a.heads
    fl = 2.0 * a.batch * a.seq * a.embed * 4 * a.embed + 4.0 * a.batch * a.heads * a.seq * a.seq * D / 2
    return {"head_dim": D, "fwd_ms": f, "fwd_tflops": round(fl / f / 1e9, 1), "fwd_bwd_ms": fb, "fwd_bwd_tflops": round(3 * fl / fb / 1e9, 1)}


def cmd_conv_bn_pool(a):
    """The reference's layer-pipeline benchmark (benchmarks/pipeline_benchmark.cpp:20-62): convolution -> batch norm
    (+ ReLU) -> max pooling on a 128 x 224 x 224 x 3 batch."""
    from tnn_b200.nn import layers as L
    from tnn_b200.nn.graph import Graph

    g = Graph()
    h = L.Conv2D(3, a.cout, 3, 3, 1, 1, 1, 1, name="conv")(g.input("input"))
    h = L.BatchNorm(a.cout, use_relu=True, name="bn")(h)
    out = L.MaxPool2D(2, 2, 2, 2, name="pool")(h)
    out.set_uid("output")
    g.set_output(out)
    g.compile(device="cuda", seed=0)
    x = bf(a.batch, a.size, a.size, 3)
    f, fb = _time_graph(g, x, a.iters)
    act = a.batch * a.size * a.size * a.cout * 2  # bytes of the convolution output
    return {"fwd_ms": f, "fwd_bwd_ms": fb, "conv_output_mb": round(act / 1e6, 1), "images_per_s_fwd_bwd": round(a.batch / fb * 1e3, 1)}


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("gemm"); p.add_argument("--m", type=int, default=8192); p.add_argument("--n", type=int, default=3072)
    p.add_argument("--k", type=int, default=768); p.add_argument("--bn", type=int, default=0); p.add_argument("--all", action="store_true")
    p = sub.add_parser("attention"); p.add_argument("--batch", type=int, default=8); p.add_argument("--heads", type=int, default=12)
    p.add_argument("--seq", type=int, default=1024); p.add_argument("--library", action="store_true")
    p = sub.add_parser("layernorm"); p.add_argument("--rows", type=int, default=65536); p.add_argument("--cols", type=int, default=768)
    p = sub.add_parser("softmax_ce"); p.add_argument("--rows", type=int, default=8192); p.add_argument("--vocab", type=int, default=50257)
    p = sub.add_parser("colsum"); p.add_argument("--rows", type=int, default=8192); p.add_argument("--cols", type=int, default=3072)
    p = sub.add_parser("adam"); p.add_argument("--n", type=int, default=163_000_000)
    p = sub.add_parser("conv2d"); p.add_argument("--batch", type=int, default=128); p.add_argument("--size", type=int, default=56)
    p.add_argument("--cin", type=int, default=64); p.add_argument("--cout", type=int, default=64); p.add_argument("--ksize", type=int, default=3)
    p.add_argument("--stride", type=int, default=1); p.add_argument("--library", action="store_true")
    p = sub.add_parser("conv_table"); p.add_argument("--batch", type=int, default=256)
    p = sub.add_parser("attention_block"); p.add_argument("--batch", type=int, default=16); p.add_argument("--seq", type=int, default=512)
    p.add_argument("--embed", type=int, default=768); p.add_argument("--heads", type=int, default=8)
    p = sub.add_parser("conv_bn_pool"); p.add_argument("--batch", type=int, default=128); p.add_argument("--size", type=int, default=224)
    p.add_argument("--cout", type=int, default=64)
    p = sub.add_parser("batchnorm"); p.add_argument("--batch", type=int, default=128); p.add_argument("--size", type=int, default=56)
    p.add_argument("--channels", type=int, default=256)
    for sp in sub.choices.values():
        sp.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    res = globals()["cmd_" + a.cmd](a)
    _lib.check_status()
    print(json.dumps({"bench": a.cmd, "args": {k: v for k, v in vars(a).items() if k != "cmd"},
                      **{k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}}))


if __name__ == "__main__":
    main()
