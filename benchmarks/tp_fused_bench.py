"""Fused tensor-parallel hand-offs against their NCCL baselines, device-timed (CUDA-graph replay of 20 calls, max
over ranks). Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/tp_fused_bench.py

Shapes are those of GPT-2 small with 16 sequences of 1024 tokens per tensor-parallel pair. A hand-off is timed
together with the layer norm it rides on, in three forms:

    fused   layer norm that also sends its rows to the peers -> all-gather GEMM   |  GEMM that pushes partial sums -> layer norm that pulls
    nccl    layer norm -> all_gather -> GEMM                           |  GEMM -> reduce_scatter -> layer norm
    local   layer norm -> GEMM on an already complete operand          |  GEMM -> layer norm (no communication at all)

`local` is what the same kernels cost with the communication removed; fused - local is the exposed cost of the
hand-off. Roofline of a hand-off = max(GEMM FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s); the
fraction printed is roofline / (fused - layer norm alone). Successive replays reuse the same buffers without the
dependencies a training step has between them; the values written are identical on every replay."""
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
local=int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda",local))
from tnn_b200.parallel.runtime import Topology
from tnn_b200.parallel.symm import SymmetricHeap
from tnn_b200.parallel.tp import CommContext, GatherSite, ScatterSite
from tnn_b200.ops import _lib, raw
from tnn_b200.ops.gemm import gemm
tp = dist.get_world_size()
topo = Topology(f"tp{tp}")
dev = torch.device("cuda", local)
heap = SymmetricHeap(2 << 30, None, dev)
cc = CommContext(topo, heap, True, dev)   # TNNB_TP_PUSH selects who sends the rows (ln, gemm, split)
cn = CommContext(topo, None, False, dev)
PEAK = 1393.6e12  # measured sustained cuBLAS bf16 rate of this pool (MEASURED_PEAKS.json); burst 1681.9e12
LINK = 770e9      # measured peer-copy bandwidth per direction
def bf(*s): return (torch.randn(*s, device=dev) * 0.5).bfloat16()
def timeit(fn, it=20):
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
    best = 1e9
    for _ in range(3):
        s=torch.cuda.Event(enable_timing=True); e=torch.cuda.Event(enable_timing=True)
        dist.barrier(); torch.cuda.synchronize()
        s.record(); g.replay(); e.record(); torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)/it], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); best = min(best, t.item()*1e3)
    return best
M, E = 8192 * tp, 768
rows = M // tp
out = []
x = bf(rows, E); gamma, beta = bf(E) + 1, bf(E)
t_ln = timeit(lambda: raw.layernorm_fwd(x, None, gamma, beta, 1e-5))
for name, N in (("QKV", 3 * E // tp), ("fc1", 4 * E // tp)):
    ctr = cc.new_pass_counter(); site = GatherSite(cc, M, E, ctr); site_n = GatherSite(cn, M, E); w = bf(N, E)
    def fused():
        ctr.add_(1); raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=site.mine(), tp_push=site.push_args())
        y = site.gemm(w); return y
    def nccl():
        raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=site_n.mine()); return site_n.gemm(w)
    full = bf(M, E)
    def loc():
        raw.layernorm_fwd(x, None, gamma, beta, 1e-5); return gemm(full, w)
    tf = timeit(fused); _lib.check_status(); tn = timeit(nccl); tl = timeit(loc); tg = timeit(lambda: gemm(full, w))
    bytes_link = (tp - 1) * rows * E * 2
    roof = max(2.0 * M * N * E / PEAK, bytes_link / LINK) * 1e6
    out.append({"op": f"all-gather -> GEMM ({name}) N={N} K={E}", "fused_us": tf, "nccl_us": tn, "local_us": tl, "gemm_us": tg, "ln_us": t_ln,
                "exposed_us": tf - tl, "roofline_us": roof, "frac": roof / max(tf - t_ln, 1e-3), "speedup_vs_nccl": tn / tf})
for name, K in (("attention out", E // tp), ("fc2", 4 * E // tp)):
    ctr = cc.new_pass_counter(); site = ScatterSite(cc, M, E, ctr); site_n = ScatterSite(cn, M, E); a = bf(M, K); w = bf(E, K); bias = bf(E)
    def fused():
        ctr.add_(1); p = site.gemm(a, w, bias=bias); return raw.layernorm_fwd(x, p, gamma, beta, 1e-5, tp_pull=site.pull_args())
    def nccl():
        p = site_n.gemm(a, w, bias=bias); return raw.layernorm_fwd(x, p, gamma, beta, 1e-5)
    half = bf(rows, E)
    def loc():
        gemm(a, w, bias=bias); return raw.layernorm_fwd(x, half, gamma, beta, 1e-5)
    t_ln2 = timeit(lambda: raw.layernorm_fwd(x, half, gamma, beta, 1e-5))
    tf = timeit(fused); _lib.check_status(); tn = timeit(nccl); tl = timeit(loc); tg = timeit(lambda: gemm(a, w, bias=bias))
    bytes_link = (tp - 1) * rows * E * 2
    roof = max(2.0 * M * E * K / PEAK, bytes_link / LINK) * 1e6
    out.append({"op": f"GEMM -> reduce-scatter ({name}) N={E} K={K}", "fused_us": tf, "nccl_us": tn, "local_us": tl, "gemm_us": tg, "ln_us": t_ln2,
                "exposed_us": tf - tl, "roofline_us": roof, "frac": roof / max(tf - t_ln2, 1e-3), "speedup_vs_nccl": tn / tf})
# the pieces on their own: what a push costs the kernel that carries it
ctr = cc.new_pass_counter(); site = GatherSite(cc, M, E, ctr)
def ln_push():
    raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=site.mine(), tp_push=site.push_args())
def push_only():
    site.push(x)
parts = {"ln_fwd_us": t_ln, "ln_fwd_then_push_us": timeit(ln_push),
         "push_only_us": timeit(push_only)}
# the same rows sent by the bulk-copy unit (one thread per block, shared-memory staging), checked against NCCL once
if cc.push_mode in ("ln", "split"):
    site.buf.zero_(); torch.cuda.synchronize(); dist.barrier()
    site.push(x, bulk_ctas=0); torch.cuda.synchronize(); dist.barrier()
    ref = torch.empty(M, E, dtype=x.dtype, device=dev); dist.all_gather_into_tensor(ref, x)
    parts["push_bulk_matches_nccl"] = float(torch.equal(site.buf, ref))
    _lib.check_status()
    for ctas in (148, 296, 592):
        parts[f"push_bulk_{ctas}ctas_us"] = timeit(lambda: (site.push(x, bulk_ctas=ctas)))
    # the layer-norm kernel sending its rows the same way (a staging row per warp, one bulk copy per row and peer)
    os.environ["TNNB_TP_LN_BULK"] = "1"
    site.buf.zero_(); torch.cuda.synchronize(); dist.barrier()
    ln_push(); torch.cuda.synchronize(); dist.barrier()
    mine_ref = raw.layernorm_fwd(x, None, gamma, beta, 1e-5)[1]
    ref = torch.empty(M, E, dtype=x.dtype, device=dev); dist.all_gather_into_tensor(ref, mine_ref.contiguous())
    parts["ln_bulk_matches_nccl"] = float(torch.equal(site.buf, ref))
    parts["ln_fwd_then_bulk_push_us"] = timeit(ln_push)
    ctrb = cc.new_pass_counter(); siteb = GatherSite(cc, M, E, ctrb); wq = bf(3 * E // tp, E)
    def fused_bulk():
        ctrb.add_(1); raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=siteb.mine(), tp_push=siteb.push_args())
        y = siteb.gemm(wq); return y
    parts["qkv_handoff_ln_bulk_us"] = timeit(fused_bulk); _lib.check_status()
    os.environ["TNNB_TP_LN_BULK"] = "0"
    parts["qkv_handoff_ln_stores_us"] = timeit(fused_bulk); _lib.check_status()
for K in (E // tp, 4 * E // tp):
    ctr2 = cc.new_pass_counter(); s2 = ScatterSite(cc, M, E, ctr2); a = bf(M, K); w = bf(E, K)
    parts[f"gemm_rs_push_K{K}_us"] = timeit(lambda: s2.gemm(a, w))
    parts[f"gemm_plain_K{K}_us"] = timeit(lambda: gemm(a, w))
parts["bytes_pushed_MB"] = (tp - 1) * rows * E * 2 / 1e6
if dist.get_rank() == 0:
    print(json.dumps({k: round(v, 2) for k, v in parts.items()}), flush=True)
    for r in out:
        print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()}), flush=True)
torch.cuda.synchronize(); dist.barrier()
heap.close(); dist.destroy_process_group()
