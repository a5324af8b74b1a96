"""Worker of the 2-GPU kernel-level tensor-parallel tests (one rank per GPU, launched through torch.distributed.run).

Runs the fused hand-offs across real GPUs - layer norm that pushes its rows -> all-gather GEMM, and GEMM that
pushes partial sums -> layer norm that pulls them - and compares every result with an fp32 computation on the
operands gathered through NCCL and with the NCCL path of the same site classes (``fused=False``)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.ops import _lib, raw  # noqa: E402
from tnn_b200.parallel.runtime import Topology  # noqa: E402
from tnn_b200.parallel.symm import SymmetricHeap  # noqa: E402
from tnn_b200.parallel.tp import CommContext, GatherSite, ScatterSite  # noqa: E402


def gather(x, tp):
    parts = [torch.empty_like(x) for _ in range(tp)]
    dist.all_gather(parts, x.contiguous())
    return parts


def err(got, ref):
    got, ref = got.float(), ref.float()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-6)), bool(torch.allclose(got, ref, rtol=3e-2, atol=3e-2 * float(ref.abs().max())))


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    tp = dist.get_world_size()
    rank = dist.get_rank()
    topo = Topology(f"tp{tp}")
    heap = SymmetricHeap(512 << 20, None, dev)
    cc = CommContext(topo, heap, True, dev)
    if len(sys.argv) > 1:
        cc.push_mode = sys.argv[1]  # "ln" (default), "split" or "gemm": see CommContext.push_mode
    cn = CommContext(topo, None, False, dev)  # NCCL path of the same classes
    torch.manual_seed(1000 + rank)
    res = {}

    def bf(*s, scale=1.0):
        return (torch.randn(*s, device=dev) * scale).bfloat16()

    worst, all_ok = 0.0, True
    for (M, K, N, b_t) in ((2048, 256, 328, False), (1024, 128, 203 * 8, False), (2048, 256, 384, True), (512, 768, 1152, False)):
        rows = M // tp
        ctr = cc.new_pass_counter()
        site, site_n = GatherSite(cc, M, K, ctr), GatherSite(cn, M, K)
        torch.manual_seed(7)  # weights are replicated
        gamma, beta = bf(K, scale=0.5) + 1, bf(K, scale=0.1)
        w = bf(K, N, scale=0.2) if b_t else bf(N, K, scale=0.2)
        bias = bf(N, scale=0.3)
        torch.manual_seed(1000 + rank + M)
        for it in range(3):
            x = bf(rows, K)
            ctr.add_(1)
            raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=site.mine(), tp_push=site.push_args())
            y = site.gemm(w, b_t=b_t, bias=bias)
            raw.layernorm_fwd(x, None, gamma, beta, 1e-5, h_out=site_n.mine())
            y_n = site_n.gemm(w, b_t=b_t, bias=bias)
            xs = torch.cat(gather(x, tp)).float()
            mu, var = xs.mean(1, keepdim=True), xs.var(1, unbiased=False, keepdim=True)
            h = ((xs - mu) * torch.rsqrt(var + 1e-5) * gamma.float() + beta.float()).bfloat16().float()
            ref = h @ (w.float() if b_t else w.float().t()) + bias.float()
            for name, got, want in (("ag_vs_fp32", y, ref), ("ag_vs_nccl", y, y_n), ("ag_buf", site.buf, h)):
                e, ok = err(got, want)
                worst, all_ok = max(worst, e), all_ok and ok
            # a site may be written again only after every rank has finished reading it; a training step has the
            # dependencies between its kernels for that, this loop needs a barrier
            torch.cuda.synchronize()
            dist.barrier()
        _lib.check_status()
    res["ag_worst"] = worst
    res["ag_ok"] = all_ok

    worst, all_ok = 0.0, True
    for (M, K, N, b_t) in ((2048, 192, 256, False), (1024, 64, 328, False), (2048, 384, 768, True), (512, 1536, 768, False)):
        rows = M // tp
        ctr = cc.new_pass_counter()
        site, site_n = ScatterSite(cc, M, N, ctr), ScatterSite(cn, M, N)
        torch.manual_seed(11)
        gamma, beta = bf(N, scale=0.5) + 1, bf(N, scale=0.1)
        bias = bf(N, scale=0.3)
        torch.manual_seed(2000 + rank + M)
        for it in range(3):
            a = bf(M, K)
            w = bf(K, N, scale=0.2) if b_t else bf(N, K, scale=0.2)
            x = bf(rows, N)
            ctr.add_(1)
            part = site.gemm(a, w, b_t=b_t, bias=bias)
            xo, h, _, _ = raw.layernorm_fwd(x, part, gamma, beta, 1e-5, tp_pull=site.pull_args())
            red = site.resolve(part)
            full_n = site_n.gemm(a, w, b_t=b_t, bias=bias)  # NCCL reduce-scatter + bias
            prod = a.float() @ (w.float() if b_t else w.float().t())
            dist.all_reduce(prod)
            mine = prod[rank * rows:(rank + 1) * rows] + bias.float()
            for name, got, want in (("rs_vs_fp32", red, mine), ("rs_vs_nccl", red, full_n), ("rs_ln_x", xo, x.float() + mine)):
                e, ok = err(got, want)
                worst, all_ok = max(worst, e), all_ok and ok
            torch.cuda.synchronize()
            dist.barrier()
        _lib.check_status()
    res["rs_worst"] = worst
    res["rs_ok"] = all_ok
    flags = torch.tensor([int(res["ag_ok"]), int(res["rs_ok"])], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    res["all_ranks_ok"] = bool(flags.min().item())
    w = torch.tensor([res["ag_worst"], res["rs_worst"]], device=dev)
    dist.all_reduce(w, op=dist.ReduceOp.MAX)
    res["ag_worst"], res["rs_worst"] = float(w[0]), float(w[1])
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        print("WORKER-ERROR rank", os.environ.get("RANK"), traceback.format_exc()[-1500:].replace("\n", " | "), flush=True)
        os._exit(1)
