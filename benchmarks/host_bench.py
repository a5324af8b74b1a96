#!/usr/bin/env python
"""Host-side benchmarks that mirror the reference's small benchmark programs.

    python benchmarks/host_bench.py serialization [--mib 128]   # wire-format message encode / packetise / reassemble / parse
    python benchmarks/host_bench.py tnng [--model cifar10_resnet9]  # checkpoint write + read throughput
    python benchmarks/host_bench.py grad_clear [--model gpt2_small] # per-tensor fill vs one memset over the gradient slab
    python benchmarks/host_bench.py memcpy [--mib 256]           # pinned / pageable host<->device copies (needs a GPU)
    python benchmarks/host_bench.py tcp [--mib 128] [--seconds 10] [--peer host:port]  # ping-pong over the TCP communicator

Reference counterparts: benchmarks/serialization_benchmark.cpp, benchmarks/grad_clear_benchmark.cpp:7-54 (per-tensor
fill against a slab memset on gpt2_small), benchmarks/memcpy_benchmark.cpp, and the 128 MiB message of
benchmarks/tcp_communicator_benchmark.cpp:132-223 (256 x 32 x 32 x 128 fp32). Each command prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.host import H  # noqa: E402
from tnn_b200.io import tnng  # noqa: E402
from tnn_b200.models import zoo  # noqa: E402
from tnn_b200.parallel.stage_worker import job_message  # noqa: E402


def best(fn, reps=5):
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return min(ts)


def cmd_serialization(a):
    n = a.mib * (1 << 20) // 4
    t = torch.randn(n // (32 * 32 * 128), 32, 32, 128) if n >= 32 * 32 * 128 else torch.randn(n)
    nbytes = t.numel() * 4
    msg = job_message("FORWARD_JOB", 7, {"activation": t})
    enc = best(lambda: job_message("FORWARD_JOB", 7, {"activation": t}))
    packets = H.slice_message(msg, 99, a.packet_mib << 20)
    slc = best(lambda: H.slice_message(msg, 99, a.packet_mib << 20))

    def reassemble():
        agg = H.Aggregator()
        out = None
        for p in packets:
            done = agg.feed(p)
            if done is not None:
                out = done[1]
        return out

    whole = reassemble()
    assert whole is not None and bytes(whole) == bytes(msg)
    agg_t = best(reassemble)
    dec = best(lambda: H.parse_message(msg))
    back = dict(H.parse_message(msg)["job"]["tensors"])["activation"]
    assert torch.equal(tnng.record_to_tensor(back), t)
    gb = nbytes / 1e9
    return {"bench": "serialization", "message_mib": round(len(msg) / 2 ** 20, 1), "packets": len(packets),
            "encode_gbs": round(gb / enc, 2), "slice_gbs": round(gb / slc, 2), "reassemble_gbs": round(gb / agg_t, 2),
            "parse_gbs": round(gb / dec, 2)}


def cmd_tnng(a):
    g = zoo.create(a.model).compile(device="cpu", seed=0)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.tnng")
        w = best(lambda: g.save_state(path), 3)
        size = os.path.getsize(path)
        r = best(lambda: tnng.read_file(path), 3)
    return {"bench": "tnng", "model": a.model, "file_mib": round(size / 2 ** 20, 1), "write_gbs": round(size / 1e9 / w, 2),
            "read_gbs": round(size / 1e9 / r, 2)}


def cmd_grad_clear(a):
    dev = "cuda" if torch.cuda.is_available() and not a.cpu else "cpu"
    g = zoo.create(a.model).compile(device=dev, seed=0)
    grads = [x for x in g.gradients() if x is not None]

    def sync():
        if dev == "cuda":
            torch.cuda.synchronize()

    def per_tensor():
        for x in grads:
            x.zero_()
        sync()

    def slab():
        g.zero_grads()
        sync()

    per_tensor(), slab()
    tp, ts = best(per_tensor, 10), best(slab, 10)
    nbytes = g.grads_flat.numel() * g.grads_flat.element_size()
    return {"bench": "grad_clear", "model": a.model, "device": dev, "tensors": len(grads), "slab_mib": round(nbytes / 2 ** 20, 1),
            "per_tensor_ms": round(tp * 1e3, 3), "slab_memset_ms": round(ts * 1e3, 3), "speedup": round(tp / ts, 2),
            "slab_gbs": round(nbytes / 1e9 / ts, 1)}


def cmd_memcpy(a):
    if not torch.cuda.is_available():
        return {"bench": "memcpy", "unavailable": "needs a GPU"}
    n = a.mib << 20
    dev = torch.empty(n, dtype=torch.uint8, device="cuda")
    out = {"bench": "memcpy", "mib": a.mib}
    for name, host in (("pinned", torch.empty(n, dtype=torch.uint8).pin_memory()), ("pageable", torch.empty(n, dtype=torch.uint8))):
        def h2d():
            dev.copy_(host, non_blocking=True)
            torch.cuda.synchronize()

        def d2h():
            host.copy_(dev, non_blocking=True)
            torch.cuda.synchronize()

        h2d(), d2h()
        out[f"{name}_h2d_gbs"] = round(n / 1e9 / best(h2d), 1)
        out[f"{name}_d2h_gbs"] = round(n / 1e9 / best(d2h), 1)
    d2 = torch.empty_like(dev)

    def d2d():
        d2.copy_(dev)
        torch.cuda.synchronize()

    d2d()
    out["d2d_gbs"] = round(2 * n / 1e9 / best(d2d), 1)
    return out


def cmd_tcp(a):
    """Ping-pong of one large message with an echoing peer (reference: benchmarks/tcp_communicator_benchmark.cpp:132-223,
    128 MiB messages for 10 s, MB/s). Without ``--peer`` the echo process is started on this host (loopback)."""
    import subprocess

    from tnn_b200.parallel.stage_worker import simple_message
    from tnn_b200.parallel.tcp_transport import TcpTransport, ping_pong

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc, peer = None, a.peer
    if not peer:
        proc = subprocess.Popen([sys.executable, "-m", "tnn_b200.parallel.tcp_transport", "echo", "--sockets", str(a.sockets),
                                 "--max-packet", str(a.packet_mib << 20)], stdout=subprocess.PIPE, text=True, cwd=root,
                                env=dict(os.environ, PYTHONPATH=root))
        peer = proc.stdout.readline().split()[1]
    t = TcpTransport(a.host, 0, a.sockets, a.packet_mib << 20)
    try:
        ping_pong(t, peer, 1 << 20, 0.2)  # connect and warm up
        r = ping_pong(t, peer, a.mib << 20, a.seconds)
        small = ping_pong(t, peer, 6, min(a.seconds, 2.0))
        t.send(peer, simple_message("SHUTDOWN"))
    finally:
        t.close()
        if proc is not None:
            proc.wait(timeout=30)
    return {"bench": "tcp_ping_pong", "peer": peer, "message_mib": a.mib, "sockets": a.sockets, "packet_mib": a.packet_mib,
            "round_trips": r["round_trips"], "mb_per_s_each_way": round(r["mb_per_s_each_way"], 1),
            "small_message_round_trip_us": round(small["seconds"] / max(1, small["round_trips"]) * 1e6, 1)}


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serialization")
    s.add_argument("--mib", type=int, default=128)
    s.add_argument("--packet-mib", type=int, default=4)
    s = sub.add_parser("tnng")
    s.add_argument("--model", default="cifar10_resnet9")
    s = sub.add_parser("grad_clear")
    s.add_argument("--model", default="gpt2_small")
    s.add_argument("--cpu", action="store_true")
    s = sub.add_parser("memcpy")
    s.add_argument("--mib", type=int, default=256)
    s = sub.add_parser("tcp")
    s.add_argument("--mib", type=int, default=128)
    s.add_argument("--seconds", type=float, default=10.0)
    s.add_argument("--sockets", type=int, default=4)
    s.add_argument("--packet-mib", type=int, default=4)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--peer", default="", help="host:port of a running `python -m tnn_b200.parallel.tcp_transport echo`")
    a = ap.parse_args()
    print(json.dumps({"tcp": cmd_tcp, "serialization": cmd_serialization, "tnng": cmd_tnng, "grad_clear": cmd_grad_clear, "memcpy": cmd_memcpy}[a.cmd](a)))


if __name__ == "__main__":
    main()
