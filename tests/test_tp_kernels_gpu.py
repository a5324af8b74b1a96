"""Numerics of the tensor-parallel hand-off kernels on ONE GPU.

The ranks of a tensor-parallel group are emulated as separate sets of buffers on one device, and their kernels
run one after the other on one stream in an order in which every producer precedes its consumer (all pushes of a
hand-off, then all consumers). No kernel therefore ever waits for a launch that has not happened yet: every poll
finds its counter already at the target. What is checked is the data path - peer stores, inbox sums, counters,
tile order, epilogues - against fp32 references; the same kernels across real GPUs are covered by
test_parallel_gpu.py.
"""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from tnn_b200.ops import _lib, raw
    from tnn_b200.parallel.tp import CommContext, GatherSite, ScatterSite


class _VirtualHeap:
    """Allocation number k of every emulated rank is its own tensor; ``peer_ptrs`` lists all ranks' copies."""

    def __init__(self, tp, dev):
        self.tp, self.dev, self.allocs = tp, dev, []

    def view(self, r):
        return _HeapView(self, r)


class _HeapView:
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


def _contexts(tp, dev, push_mode="ln"):
    heap = _VirtualHeap(tp, dev)
    ccs = []
    for r in range(tp):
        topo = types.SimpleNamespace(tp=tp, tp_idx=r, tp_ranks=list(range(tp)), tp_group=None)
        cc = CommContext(topo, heap.view(r), True, dev)
        cc.push_mode = push_mode
        ccs.append(cc)
    return ccs


def _bf(*shape, scale=1.0, dev="cuda"):
    return (torch.randn(*shape, device=dev) * scale).bfloat16()


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got, ref = got.float(), ref.float()
    assert torch.allclose(got, ref, rtol=rtol, atol=atol * max(1.0, float(ref.abs().max()))), \
        f"max err {float((got - ref).abs().max()):.4f} vs max ref {float(ref.abs().max()):.3f}"


def _ln_ref(x, gamma, beta, eps=1e-5):
    x = x.float()
    m, v = x.mean(1, keepdim=True), x.var(1, unbiased=False, keepdim=True)
    return (x - m) * torch.rsqrt(v + eps) * gamma.float() + beta.float()


@pytest.mark.parametrize("mode", ["ln", "lnbulk"])  # "gemm" needs the ranks' kernels to run at the same time: 2-GPU tests
@pytest.mark.parametrize("tp,M,K,N,b_t", [(2, 1024, 256, 320, False), (2, 256, 128, 72, False), (2, 1024, 256, 384, True),
                                           (4, 2048, 128, 256, False)])
def test_layernorm_push_then_gather_gemm(tp, M, K, N, b_t, mode, monkeypatch):
    """``ln``: the layer-norm kernel stores its rows into the peers' buffers itself (``lnbulk``: through shared
    memory with bulk copies)."""
    torch.manual_seed(0)
    dev = torch.device("cuda")
    monkeypatch.setenv("TNNB_TP_LN_BULK", "1" if mode == "lnbulk" else "0")
    mode = "ln" if mode == "lnbulk" else mode
    ccs = _contexts(tp, dev, mode)
    ctrs = [cc.new_pass_counter() for cc in ccs]
    sites = [GatherSite(cc, M, K, c) for cc, c in zip(ccs, ctrs)]
    rows = M // tp
    gamma, beta = _bf(K, scale=0.5) + 1, _bf(K, scale=0.1)
    w = _bf(K, N, scale=0.2) if b_t else _bf(N, K, scale=0.2)
    bias = _bf(N, scale=0.3)
    for it in range(2):  # two passes in a row: the counters accumulate
        xs = [_bf(rows, K) for _ in range(tp)]
        for c in ctrs:
            c.add_(1)
        for r in range(tp):
            raw.layernorm_fwd(xs[r], None, gamma, beta, 1e-5, h_out=sites[r].mine(), tp_push=sites[r].push_args())
        outs = [sites[r].gemm(w, b_t=b_t, bias=bias) for r in range(tp)]
        _lib.check_status()
        h = torch.cat([_ln_ref(x, gamma, beta) for x in xs]).bfloat16().float()
        ref = h @ (w.float() if b_t else w.float().t()) + bias.float()
        for r in range(tp):
            _close(sites[r].buf, h)      # every rank holds the full gathered operand afterwards
            _close(outs[r], ref)
    for r in range(tp):  # counters: two passes of 128 rows for every block a peer owns, nothing for the own blocks
        cnt = sites[r].ready[:M // 128].view(tp, -1)
        for o in range(tp):
            assert int(cnt[o].min()) == int(cnt[o].max()) == (0 if o == r else 256), (r, o, cnt[o])


@pytest.mark.parametrize("tp,M,K,ctas", [(2, 1024, 256, 0), (2, 2048, 768, 7), (4, 1024, 128, 0)])
def test_bulk_push_delivers_rows_and_counts(tp, M, K, ctas):
    """Stand-alone push through the bulk-copy unit: every rank's buffer ends up complete and every 128-row block a
    peer owns has been counted once per row."""
    torch.manual_seed(3)
    dev = torch.device("cuda")
    ccs = _contexts(tp, dev, "ln")
    sites = [GatherSite(cc, M, K, cc.new_pass_counter()) for cc in ccs]
    rows = M // tp
    for it in range(2):
        xs = [_bf(rows, K) for _ in range(tp)]
        for r in range(tp):
            sites[r].push(xs[r], bulk_ctas=ctas)
        torch.cuda.synchronize()
        _lib.check_status()
        full = torch.cat(xs)
        for r in range(tp):
            assert torch.equal(sites[r].buf, full)
    for r in range(tp):
        cnt = sites[r].ready[:M // 128].view(tp, -1)
        for o in range(tp):
            assert int(cnt[o].min()) == int(cnt[o].max()) == (0 if o == r else 256), (r, o, cnt[o])


def test_gather_gemm_gelu_epilogues():
    torch.manual_seed(1)
    dev = torch.device("cuda")
    tp, M, K, N = 2, 512, 128, 256
    ccs = _contexts(tp, dev)
    ctrs = [cc.new_pass_counter() for cc in ccs]
    sites = [GatherSite(cc, M, K, c) for cc, c in zip(ccs, ctrs)]
    rows = M // tp
    xs = [_bf(rows, K) for _ in range(tp)]
    w, bias = _bf(N, K, scale=0.2), _bf(N, scale=0.3)
    for c in ctrs:
        c.add_(1)
    for r in range(tp):
        sites[r].push(xs[r])  # stand-alone push
    full = torch.cat(xs).float()
    pre = full @ w.float().t() + bias.float()
    for r in range(tp):
        z = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        y = sites[r].gemm(w, bias=bias, gelu_preact=z)
        _close(z, pre)
        _close(y, torch.nn.functional.gelu(z.float(), approximate="tanh"))
    # backward-style: times GELU'(z)
    for c in ctrs:
        c.add_(1)
    for r in range(tp):
        sites[r].push(xs[r])
    zsave = pre.bfloat16()
    t = zsave.float().requires_grad_(True)
    torch.nn.functional.gelu(t, approximate="tanh").sum().backward()
    for r in range(tp):
        y = sites[r].gemm(w, dgelu_of=zsave)
        _close(y, (full @ w.float().t()) * t.grad)
    _lib.check_status()


@pytest.mark.parametrize("tp,M,K,N,b_t", [(2, 1024, 192, 256, False), (2, 256, 64, 328, False), (2, 512, 128, 768, True),
                                           (4, 1024, 64, 128, False)])
def test_scatter_gemm_then_layernorm_pull(tp, M, K, N, b_t):
    torch.manual_seed(2)
    dev = torch.device("cuda")
    ccs = _contexts(tp, dev)
    ctrs = [cc.new_pass_counter() for cc in ccs]
    sites = [ScatterSite(cc, M, N, c) for cc, c in zip(ccs, ctrs)]
    rows = M // tp
    gamma, beta = _bf(N, scale=0.5) + 1, _bf(N, scale=0.1)
    bias = _bf(N, scale=0.3)
    for it in range(2):
        a = [_bf(M, K) for _ in range(tp)]
        w = [(_bf(K, N, scale=0.2) if b_t else _bf(N, K, scale=0.2)) for _ in range(tp)]
        x = [_bf(rows, N) for _ in range(tp)]
        for c in ctrs:
            c.add_(1)
        part = [sites[r].gemm(a[r], w[r], b_t=b_t, bias=bias) for r in range(tp)]
        total = sum(a[r].float() @ (w[r].float() if b_t else w[r].float().t()) for r in range(tp)) + bias.float()
        for r in range(tp):
            mine = total[r * rows:(r + 1) * rows]
            if N % 8 == 0:
                xo, h, mean, rstd = raw.layernorm_fwd(x[r], part[r], gamma, beta, 1e-5, tp_pull=sites[r].pull_args())
                _close(xo, x[r].float() + mine)
                _close(h, _ln_ref((x[r].float() + mine).bfloat16(), gamma, beta), atol=4e-2)
            _close(sites[r].resolve(part[r]), mine)
        _lib.check_status()


def test_layernorm_backward_pull_and_push():
    torch.manual_seed(3)
    dev = torch.device("cuda")
    tp, M, C = 2, 512, 256
    rows = M // tp
    ccs = _contexts(tp, dev)
    cb = [cc.new_pass_counter() for cc in ccs]
    scat = [ScatterSite(cc, M, C, c) for cc, c in zip(ccs, cb)]
    gath = [GatherSite(cc, M, C, c) for cc, c in zip(ccs, cb)]
    gamma = _bf(C, scale=0.5) + 1
    for c in cb:
        c.add_(1)
    # partial sums of dh arrive through a reduce-scatter GEMM with identity-like weights
    a = [_bf(M, 64) for _ in range(tp)]
    w = [_bf(C, 64, scale=0.2) for _ in range(tp)]
    part = [scat[r].gemm(a[r], w[r]) for r in range(tp)]
    dh_full = sum(a[r].float() @ w[r].float().t() for r in range(tp))
    xs = [_bf(rows, C) for _ in range(tp)]
    dres = [_bf(rows, C) for _ in range(tp)]
    dd_all = []
    for r in range(tp):
        mean = xs[r].float().mean(1)
        rstd = torch.rsqrt(xs[r].float().var(1, unbiased=False) + 1e-5)
        dg = torch.zeros(C, device=dev)
        db = torch.zeros(C, device=dev)
        dx, dd = raw.layernorm_bwd(part[r], xs[r], mean, rstd, gamma, dres[r], True, 0.0, 0, dg, db,
                                   ddelta_out=gath[r].mine(), tp_pull=scat[r].pull_args(), tp_push=gath[r].push_args())
        dh = dh_full[r * rows:(r + 1) * rows].bfloat16()
        dx_ref, _ = raw.layernorm_bwd(dh.cpu().float(), xs[r].cpu().float(), mean.cpu(), rstd.cpu(), gamma.cpu().float(),
                                      dres[r].cpu().float(), True, 0.0, 0, None, None)
        _close(dx, dx_ref.to(dev), atol=4e-2)
        assert dd.data_ptr() == gath[r].mine().data_ptr()
        dd_all.append(dx.clone())
        _close(db, dh.float().sum(0), atol=4e-2)
    torch.cuda.synchronize()
    for r in range(tp):  # every rank's gather buffer holds all ranks' ddelta rows
        _close(gath[r].buf, torch.cat(dd_all))
    # and a gather GEMM over them sees the pushed rows
    wq = _bf(128, C, scale=0.2)
    for r in range(tp):
        _close(gath[r].gemm(wq), torch.cat(dd_all).float() @ wq.float().t())
    _lib.check_status()
