"""Data-parallel optimizer step in isolation: the fused kernel (peer-memory gradient reduction + AdamW on the rank's
slice + parameter broadcast, ``tnnb_dp_step``) against the library path (NCCL reduce-scatter, local AdamW kernel, NCCL
all-gather). Device-timed with CUDA events, max over ranks. One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/dp_step_bench.py [--params 163000000]

Prints one JSON line with both times, the bytes each rank moves over NVLink (reads of the other ranks' fp32 gradients
for its slice, writes of its bf16 slice to the other ranks) and the roofline fraction against ``--link-gbs``
(default 770 GB/s per direction, the peer-copy rate measured on this pool; 900 nominal).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.nn.optim import AdamW  # noqa: E402
from tnn_b200.ops import _lib, raw  # noqa: E402
from tnn_b200.parallel.dp import FusedDPOptimizer, Region  # noqa: E402
from tnn_b200.parallel.symm import SymmetricHeap  # noqa: E402


class FlatGraph:
    """The part of a compiled graph the optimizer touches: flat fp32 master / gradient slabs and the bf16 copy."""

    def __init__(self, n, heap, dev):
        self.total_elems = n
        self.params_flat = heap.alloc((n,), torch.bfloat16).zero_()
        self.grads_flat = heap.alloc((n,), torch.float32).normal_()
        self.master_flat = torch.randn(n, device=dev)
        self.trainable_mask = torch.ones(n, dtype=torch.bool, device=dev)
        self.layer_slices = {0: [(0, n, (n,), True)]}
        self.training = True
        self.grad_hook = None

    def grad_hook_usable(self):
        return False


def timeit(fn, iters, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=163_000_000)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    n = a.params // (8 * world) * (8 * world)
    heap = SymmetricHeap(n * 6 + (64 << 20), None, dev)
    g = FlatGraph(n, heap, dev)
    opt = AdamW(3e-4, 0.9, 0.95, 1e-8, 0.1)
    fused = FusedDPOptimizer(opt, g, heap, [Region(0, n, list(range(world)), None)], 1.0 / world)
    t_fused = timeit(fused.update, a.iters, dev)
    _lib.check_status(dev)
    # library path: reduce-scatter, AdamW on the slice, all-gather of the bf16 slice
    per = n // world
    shard_g = torch.empty(per, device=dev)
    m, v = torch.zeros(per, device=dev), torch.zeros(per, device=dev)
    master = g.master_flat[rank * per:(rank + 1) * per]
    lp = torch.empty(per, device=dev, dtype=torch.bfloat16)
    full_lp = torch.empty(n, device=dev, dtype=torch.bfloat16)

    def nccl_step():
        dist.reduce_scatter_tensor(shard_g, g.grads_flat)
        raw.adam_step(master, lp, shard_g, m, v, 3e-4, 0.9, 0.95, 1e-8, 0.1, 1, 1.0 / world)
        dist.all_gather_into_tensor(full_lp, lp)

    t_nccl = timeit(nccl_step, a.iters, dev)
    in_bytes = (world - 1) * per * 4          # other ranks' gradients of my slice
    out_bytes = (world - 1) * per * 2         # my updated bf16 slice to the other ranks
    hbm_bytes = per * (4 + 30)                # own gradient slice + AdamW traffic on the slice
    roof_ms = max(in_bytes, out_bytes) / (a.link_gbs * 1e9) * 1e3 if world > 1 else hbm_bytes / 6.4e12 * 1e3
    if rank == 0:
        print(json.dumps({"bench": "dp_step", "world": world, "params": n, "fused_ms": round(t_fused, 3), "nccl_ms": round(t_nccl, 3),
                          "nvlink_in_mb_per_rank": round(in_bytes / 1e6, 1), "nvlink_out_mb_per_rank": round(out_bytes / 1e6, 1),
                          "roofline_ms": round(roof_ms, 3), "fused_fraction_of_roofline": round(roof_ms / t_fused, 3),
                          "nccl_fraction_of_roofline": round(roof_ms / t_nccl, 3), "link_gbs": a.link_gbs}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
