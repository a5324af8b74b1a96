"""Fused tensor-parallel kernels against their NCCL + GEMM baselines, device-timed (CUDA-graph replay of 20 calls,
max over ranks). Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/tp_fused_bench.py

Shapes are those of GPT-2 small with 16 sequences of 1024 tokens per tensor-parallel pair: all-gather -> GEMM for the
QKV and fc1 projections, GEMM -> reduce-scatter for the attention output and fc2 projections."""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
local=int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda",local))
from tnn_b200.parallel.runtime import Topology
from tnn_b200.parallel.symm import SymmetricHeap
from tnn_b200.parallel.tp import CommContext, GatherSite, ScatterSite
from tnn_b200.ops import _lib
from tnn_b200.ops.gemm import gemm
topo = Topology("tp2")
dev = torch.device("cuda", local)
heap = SymmetricHeap(2 << 30, None, dev)
cc = CommContext(topo, heap, True, dev)
def bf(*s): return (torch.randn(*s, device=dev) * 0.5).bfloat16()
def timeit(fn, it=20):
    # CUDA-graph replay of `it` calls: removes the Python / launch overhead from the measurement
    for _ in range(3): fn()
    torch.cuda.synchronize(); dist.barrier()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        fn(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(it): fn()
    torch.cuda.synchronize(); dist.barrier()
    g.replay(); torch.cuda.synchronize(); dist.barrier()
    s=torch.cuda.Event(enable_timing=True); e=torch.cuda.Event(enable_timing=True)
    s.record()
    g.replay()
    e.record(); torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)/it], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); return t.item()*1e3
M, K = 16384, 768
for N in (128, 1152, 1536):
    site = GatherSite(cc, M, K); site.mine().copy_(bf(M//2, K)); w = bf(N, K)
    def f():
        cc.tick.add_(1); return site.gemm(w)
    t = timeit(f); _lib.check_status()
    a = bf(M, K); tg = timeit(lambda: gemm(a, w))
    if dist.get_rank()==0: print(f"AG-GEMM M={M} N={N} K={K}: fused {t:.1f} us | plain local GEMM {tg:.1f} us | copy bytes {M//2*K*2/1e6:.1f} MB", flush=True)
for (N, K) in ((768, 384), (768, 1536)):
    site = ScatterSite(cc, M, N); a = bf(M, K); w = bf(N, K)
    def f():
        cc.tick.add_(1); return site.gemm(a, w)
    t = timeit(f); _lib.check_status()
    tg = timeit(lambda: gemm(a, w))
    if dist.get_rank()==0: print(f"GEMM-RS M={M} N={N} K={K}: fused {t:.1f} us | plain local GEMM {tg:.1f} us | nvlink bytes {M//2*N*2/1e6:.1f} MB", flush=True)
# NCCL references
x = bf(M//2, 768); full = torch.empty(M, 768, device=dev, dtype=torch.bfloat16)
t = timeit(lambda: dist.all_gather_into_tensor(full, x))
y = bf(M, 768); out = torch.empty(M//2, 768, device=dev, dtype=torch.bfloat16)
t2 = timeit(lambda: dist.reduce_scatter_tensor(out, y))
if dist.get_rank()==0: print(f"NCCL all_gather 12.6MB/rank: {t:.1f} us ; reduce_scatter: {t2:.1f} us", flush=True)
heap.close(); dist.destroy_process_group()
