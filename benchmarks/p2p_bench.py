"""Ping-pong bandwidth between two ranks - the counterpart of the reference's communicator benchmarks
(benchmarks/tcp_communicator_benchmark.cpp:132-223, roce_communicator_benchmark.cpp): 128 MiB messages
(256 x 32 x 32 x 128 fp32) bounced for a fixed time, MB/s printed. Here the transports are NCCL point-to-point
over NVLink (what the pipeline stages use) and a direct peer-memory copy through the symmetric heap (what the
fused kernels use); a small-message latency sweep follows.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/p2p_bench.py
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(seconds: float = 3.0):
    local = int(os.environ.get("LOCAL_RANK", "0"))
    gpu = torch.cuda.is_available()
    if gpu:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    rank = dist.get_rank()
    assert dist.get_world_size() == 2, "ping-pong needs exactly two ranks"
    dev = torch.device("cuda", local) if gpu else torch.device("cpu")
    sync = torch.cuda.synchronize if gpu else (lambda: None)
    res = {}

    def pingpong(nbytes, min_seconds, max_iters=10 ** 6):
        buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=dev)
        for _ in range(2):
            if rank == 0:
                dist.send(buf, 1); dist.recv(buf, 1)
            else:
                dist.recv(buf, 0); dist.send(buf, 0)
        sync(); dist.barrier()
        t0, n = time.perf_counter(), 0
        stop = torch.zeros(1, device=dev)
        while n < max_iters:
            if rank == 0:
                dist.send(buf, 1); dist.recv(buf, 1)
            else:
                dist.recv(buf, 0); dist.send(buf, 0)
            n += 1
            if n % 8 == 0:  # rank 0 decides when to stop, both leave together
                sync()
                stop.fill_(1.0 if (time.perf_counter() - t0) > min_seconds else 0.0)
                dist.broadcast(stop, 0)
                if stop.item() > 0:
                    break
        sync()
        dt = time.perf_counter() - t0
        return 2 * n * nbytes / dt / 1e6, dt / (2 * n) * 1e6  # MB/s (both directions counted like the reference), one-way us

    mbs, _ = pingpong(256 * 32 * 32 * 128 * 4, seconds)
    res["backend"] = "nccl" if gpu else "gloo"
    res["p2p_128MiB_MBps"] = round(mbs)
    lat = {}
    for nb in (4, 4096, 1 << 20, 16 << 20):
        _, us = pingpong(nb, 0.3)
        lat[str(nb)] = round(us, 1)
    res["p2p_one_way_us"] = lat
    if gpu:
        from tnn_b200.parallel.symm import SymmetricHeap
        heap = SymmetricHeap(320 << 20, None, dev)
        t = heap.alloc(((128 << 20) // 4,), torch.float32)
        peer = heap.peer_view(t, 1 - rank)
        for _ in range(2):
            t.copy_(peer)
        sync(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            t.copy_(peer)  # pull 128 MiB from the peer's memory (copy engine / SM copy chosen by the runtime)
        e1.record(); sync()
        res["peer_memory_pull_128MiB_MBps"] = round(10 * (128 << 20) / (e0.elapsed_time(e1) / 1e3) / 1e6)
        dist.barrier()
        heap.close()
    if rank == 0:
        print(json.dumps({"bench": "p2p", **res}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
