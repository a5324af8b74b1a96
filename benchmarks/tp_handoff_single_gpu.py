"""The tensor-parallel hand-off kernels on ONE GPU, for profiling with ncu (which is never wrapped around a multi-rank
run): the two ranks of a pair are emulated as two sets of buffers on the same device and their kernels run one after
the other on one stream, every producer before its consumer, so no kernel waits for a launch that has not happened.

    python benchmarks/tp_handoff_single_gpu.py [--rows 8192] [--iters 3]
    ncu --set full --clock-control none -k regex:gemm_bf16_tcgen05_pair_kernel -s 8 -c 4 -o tp_gemm \\
        python benchmarks/tp_handoff_single_gpu.py --iters 2

Per iteration and rank: layer norm that stores its rows into the other rank's gather buffer, all-gather GEMM (QKV shape
of GPT-2 small, mode 1), reduce-scatter GEMM whose epilogue stores the other rank's partial sums into its inbox (fc2
shape, mode 2), layer norm that adds the inbox. Times are CUDA events around each kind of kernel (both ranks' launches
together); "peer" memory is local here, so the figures show the kernels' own cost, not NVLink."""
import argparse
import os
import sys
import types

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.ops import _lib, raw  # noqa: E402
from tnn_b200.ops.gemm import gemm  # noqa: E402
from tnn_b200.parallel.tp import CommContext, GatherSite, ScatterSite  # noqa: E402


class _Heap:
    def __init__(self, tp, dev):
        self.tp, self.dev, self.allocs = tp, dev, []


class _View:
    def __init__(self, heap, r):
        self.h, self.r, self.k = heap, r, 0

    def alloc(self, shape, dtype=torch.bfloat16):
        if self.k == len(self.h.allocs):
            self.h.allocs.append([torch.zeros(*shape, dtype=dtype, device=self.h.dev) for _ in range(self.h.tp)])
        t = self.h.allocs[self.k][self.r]
        self.k += 1
        return t

    def peer_ptrs(self, t, ranks=None):
        for group in self.h.allocs:
            if group[self.r].data_ptr() == t.data_ptr():
                return [g.data_ptr() for g in group]
        raise ValueError("not a heap tensor")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192, help="rows owned by each emulated rank")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda")
    tp, E = 2, 768
    M = a.rows * tp
    heap = _Heap(tp, dev)
    ccs = []
    for r in range(tp):
        topo = types.SimpleNamespace(tp=tp, tp_idx=r, tp_ranks=list(range(tp)), tp_group=None)
        cc = CommContext(topo, _View(heap, r), True, dev)
        cc.push_mode = "ln"
        ccs.append(cc)
    ctr = [cc.new_pass_counter() for cc in ccs]
    gs = [GatherSite(cc, M, E, c) for cc, c in zip(ccs, ctr)]
    ss = [ScatterSite(cc, M, E, c) for cc, c in zip(ccs, ctr)]
    bf = lambda *s: (torch.randn(*s, device=dev) * 0.5).bfloat16()  # noqa: E731
    x = [bf(a.rows, E) for _ in range(tp)]
    gamma, beta = bf(E) + 1, bf(E)
    wqkv, w2, b2 = bf(3 * E // tp, E), bf(E, 4 * E // tp), bf(E)
    act = [bf(M, 4 * E // tp) for _ in range(tp)]
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    for it in range(a.iters + 1):
        for c in ctr:
            c.add_(1)
        t = [ev() for _ in range(5)]
        t[0].record()
        for r in range(tp):
            raw.layernorm_fwd(x[r], None, gamma, beta, 1e-5, h_out=gs[r].mine(), tp_push=gs[r].push_args())
        t[1].record()
        y = [gs[r].gemm(wqkv) for r in range(tp)]
        t[2].record()
        part = [ss[r].gemm(act[r], w2, bias=b2) for r in range(tp)]
        t[3].record()
        for r in range(tp):
            raw.layernorm_fwd(x[r], part[r], gamma, beta, 1e-5, tp_pull=ss[r].pull_args())
        t[4].record()
        torch.cuda.synchronize()
        _lib.check_status()
        if it:
            d = [t[i].elapsed_time(t[i + 1]) * 1e3 / tp for i in range(4)]
            print(f"iter {it}: layer norm + push {d[0]:.1f} us | gather GEMM {d[1]:.1f} us | scatter GEMM {d[2]:.1f} us | "
                  f"layer norm + pull {d[3]:.1f} us (per rank)")
    full = torch.cat([gs[0].buf])
    ref = gemm(full, wqkv)
    err = float((y[0].float() - ref.float()).abs().max() / ref.float().abs().max())
    print("gather GEMM against the plain GEMM on the gathered operand: max rel err", err)
    assert err < 1e-2


if __name__ == "__main__":
    main()
