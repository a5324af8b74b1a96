"""Each sm_100a kernel against the fp32 torch restatement of the same op (ops.raw CPU path)."""
import pytest
import torch

from tnn_b200.ops import _lib, raw

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape) * scale).to(BF)


def close(got, ref, tol=2e-2, what=""):
    """Largest error against the largest value, and every element on its own (3 % of the element plus half of the
    first tolerance times the largest value): a kernel that drops its small elements does not pass."""
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"{what} rel err {err / scale:.4g} (abs {err:.4g})"
    bad = (got - ref).abs() > (3e-2 * ref.abs() + 0.5 * tol * scale)
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} elements outside the per-element tolerance"


@pytest.mark.parametrize("kind,alpha", [("relu", 0), ("gelu", 0), ("elu", 1.0), ("leaky_relu", 0.01),
                                        ("sigmoid", 0), ("tanh", 0), ("linear", 0)])
def test_activations(kind, alpha):
    torch.manual_seed(0)
    x, dy = rnd(1000, 37), rnd(1000, 37)
    close(raw.act_fwd(x.cuda(), kind, alpha), raw.act_fwd(x, kind, alpha), what=kind)
    close(raw.act_bwd(x.cuda(), dy.cuda(), kind, alpha), raw.act_bwd(x, dy, kind, alpha), what=kind + " bwd")


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary(op):
    a, b = rnd(333, 65), rnd(333, 65).abs() + 1
    close(raw.binary(a.cuda(), b.cuda(), op), raw.binary(a, b, op))
    close(raw.binary(a.cuda(), b.cuda(), op, relu=True), raw.binary(a, b, op, relu=True))


def test_dropout_mask_matches_host_hash():
    x = rnd(257, 129)
    y = raw.dropout(x.cuda(), 0.3, 1234567)
    ref = raw.dropout(x, 0.3, 1234567)
    close(y, ref)
    keep = (y != 0).float().mean().item()
    assert 0.6 < keep < 0.8


def test_embedding():
    torch.manual_seed(1)
    V, E, S, B = 1000, 64, 16, 3
    ids = torch.randint(0, V, (B, S))
    ids[0, 0] = V + 5  # out of range -> row 0
    wte, wpe = rnd(V, E), rnd(S, E)
    for p in (0.0, 0.1):
        o = raw.embedding_fwd(ids.cuda(), wte.cuda(), wpe.cuda(), S, V, p, 77)
        close(o, raw.embedding_fwd(ids, wte, wpe, S, V, p, 77))
        dy = rnd(B * S, E)
        g1, g2 = torch.zeros(V, E), torch.zeros(S, E)
        raw.embedding_bwd(ids, dy, g1, g2, S, V, p, 77)
        c1, c2 = torch.zeros(V, E, device="cuda"), torch.zeros(S, E, device="cuda")
        raw.embedding_bwd(ids.cuda(), dy.cuda(), c1, c2, S, V, p, 77)
        close(c1, g1, tol=1e-3)
        close(c2, g2, tol=1e-3)


@pytest.mark.parametrize("M,N", [(4096, 768), (1000, 50), (77, 3072)])
def test_colsum(M, N):
    dy = rnd(M, N)
    db = torch.ones(N, device="cuda")
    raw.colsum_accum(dy.cuda(), db)
    close(db, dy.float().sum(0) + 1, tol=1e-3)


@pytest.mark.parametrize("rows,C", [(513, 768), (64, 1024), (100, 1280), (33, 256), (10, 2048)])
@pytest.mark.parametrize("fused,p", [(False, 0.0), (True, 0.0), (True, 0.1)])
def test_layernorm(rows, C, fused, p):
    torch.manual_seed(2)
    x, d, g, b = rnd(rows, C), rnd(rows, C), rnd(C) + 1, rnd(C)
    delta = d if fused else None
    xo, h, mean, rstd = raw.layernorm_fwd(x.cuda(), None if delta is None else delta.cuda(), g.cuda(), b.cuda(), 1e-5, p, 99)
    rxo, rh, rmean, rrstd = raw.layernorm_fwd(x, delta, g, b, 1e-5, p, 99)
    close(xo, rxo, what="x_out")
    close(h, rh, what="h")
    close(mean, rmean, tol=1e-3)
    close(rstd, rrstd, tol=1e-3)
    dh, dres = rnd(rows, C), rnd(rows, C)
    dg, dbt = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    dx, dd = raw.layernorm_bwd(dh.cuda(), xo, mean, rstd, g.cuda(), dres.cuda(), fused, p, 99, dg, dbt)
    rdg, rdb = torch.zeros(C), torch.zeros(C)
    rdx, rdd = raw.layernorm_bwd(dh, rxo, rmean, rrstd, g, dres, fused, p, 99, rdg, rdb)
    close(dx, rdx, what="dx")
    if fused:
        close(dd, rdd, what="ddelta")
    close(dg, rdg, what="dgamma")
    close(dbt, rdb, what="dbeta")
    if fused:
        # the same pass with the column sums of ddelta (bias gradient of the dense layer in front of the norm),
        # accumulated onto what the buffer already holds; reference: fp32 sum of the bf16 ddelta rows
        dbias = torch.full((C,), 0.5, device="cuda")
        dg2, dbt2 = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        dx2, dd2 = raw.layernorm_bwd(dh.cuda(), xo, mean, rstd, g.cuda(), dres.cuda(), True, p, 99, dg2, dbt2, dbias=dbias)
        assert torch.equal(dx2, dx) and torch.equal(dd2, dd)
        close(dg2, rdg, what="dgamma with dbias")
        ref = 0.5 + rdd.float().sum(0)
        # the kernel sums the bf16 values it stored, in fp32: only the order of the additions differs
        err = (dbias.cpu() - 0.5 - dd.cpu().float().sum(0)).abs()
        assert bool((err <= 1e-5 * dd.cpu().float().abs().sum(0) + 1e-6).all()), err.max().item()
        close(dbias, ref, what="dbias")


@pytest.mark.parametrize("rows,V,ld", [(64, 1000, 1000), (33, 100, 104), (16, 50257, 50304), (8, 10, 10), (5, 3000, 3000)])
def test_softmax_ce(rows, V, ld):
    torch.manual_seed(3)
    buf = torch.zeros(rows, ld, dtype=BF)
    buf[:, :V] = rnd(rows, V, scale=3.0)
    labels = torch.randint(0, V, (rows,))
    logits = buf.cuda()[:, :V]
    loss, corr, grad = raw.softmax_ce(logits, labels.cuda(), V, 1.0 / rows, 1.0 / rows)
    rloss, rcorr, rgrad = raw.softmax_ce(buf[:, :V], labels, V, 1.0 / rows, 1.0 / rows)
    close(loss, rloss, tol=1e-3)
    assert int(corr.item()) == int(rcorr.item())
    close(grad, rgrad, tol=2e-2)


@pytest.mark.parametrize("B,S,H,causal", [(1, 128, 1, True), (2, 256, 3, True), (1, 384, 2, False),
                                           (2, 200, 2, True), (1, 257, 4, False), (1, 1024, 2, True)])
def test_attention_fwd_bwd(B, S, H, causal):
    torch.manual_seed(4)
    D = 64
    qkv = rnd(B * S, 3 * H * D, scale=0.7)
    scale = 0.125
    out, lse = raw.attn_fwd(qkv.cuda(), B, S, H, D, causal, scale)
    _lib.check_status()
    rout, rlse = raw.attn_fwd(qkv, B, S, H, D, causal, scale)
    close(out, rout, what="out")
    close(lse, rlse, tol=1e-2, what="lse")
    dout = rnd(B * S, H * D)
    dqkv = raw.attn_bwd(qkv.cuda(), out, dout.cuda(), lse, B, S, H, D, causal, scale)
    _lib.check_status()
    rd = raw.attn_bwd(qkv, rout, dout, rlse, B, S, H, D, causal, scale)
    E = H * D
    for i, name in enumerate("qkv"):
        close(dqkv[:, i * E:(i + 1) * E], rd[:, i * E:(i + 1) * E], tol=3e-2, what="d" + name)


@pytest.mark.parametrize("B,S,H,D,causal", [(2, 128, 2, 96, True), (1, 200, 3, 32, False), (1, 256, 1, 128, True),
                                             (3, 77, 2, 96, True), (2, 512, 8, 96, False), (1, 333, 2, 40, True)])
def test_attention_other_head_sizes(B, S, H, D, causal):
    """Head sizes other than 64 run as batched GEMMs over all heads with a row-softmax kernel between them (the
    reference's attention benchmark uses 96); sequence lengths that are no multiple of 8 or 128 included."""
    torch.manual_seed(14)
    qkv = rnd(B * S, 3 * H * D, scale=0.5)
    scale = D ** -0.5
    out, lse = raw.attn_fwd(qkv.cuda(), B, S, H, D, causal, scale)
    _lib.check_status()
    rout, rlse = raw.attn_fwd(qkv, B, S, H, D, causal, scale)
    close(out, rout, what="out")
    close(lse, rlse, tol=1e-2, what="lse")
    dout = rnd(B * S, H * D)
    dqkv = raw.attn_bwd(qkv.cuda(), out, dout.cuda(), lse, B, S, H, D, causal, scale)
    _lib.check_status()
    rd = raw.attn_bwd(qkv, rout, dout, rlse, B, S, H, D, causal, scale)
    close(dqkv, rd, tol=3e-2, what="dqkv")


def test_batched_gemm_layouts():
    """The batched tcgen05 GEMM in all four operand layouts, bf16 and fp32 output, padded output rows."""
    from tnn_b200.ops.gemm import gemm_batched
    torch.manual_seed(15)
    G, M, N, K = 5, 200, 136, 72
    for a_t in (False, True):
        for b_t in (False, True):
            a = rnd(G, K, M) if a_t else rnd(G, M, K)
            b = rnd(G, K, N) if b_t else rnd(G, N, K)
            ref = (a.transpose(1, 2) if a_t else a).float() @ (b if b_t else b.transpose(1, 2)).float()
            close(gemm_batched(a.cuda(), b.cuda(), a_t=a_t, b_t=b_t), ref, what=f"bf16 {a_t} {b_t}")
            buf = torch.zeros(G, M, 144, dtype=torch.float32, device="cuda")
            gemm_batched(a.cuda(), b.cuda(), a_t=a_t, b_t=b_t, out=buf[:, :, :N])
            close(buf[:, :, :N], ref, tol=1e-2, what=f"f32 {a_t} {b_t}")
            assert float(buf[:, :, N:].abs().max()) == 0.0
    _lib.check_status()


def test_attention_scale_one_like_reference_block():
    torch.manual_seed(5)
    B, S, H, D = 1, 256, 2, 64
    qkv = rnd(B * S, 3 * H * D, scale=0.2)
    out, _ = raw.attn_fwd(qkv.cuda(), B, S, H, D, True, 1.0)
    _lib.check_status()
    close(out, raw.attn_fwd(qkv, B, S, H, D, True, 1.0)[0])


def test_optimizers():
    torch.manual_seed(6)
    n = 100003
    w = torch.randn(n)
    g = torch.randn(n)
    for step in (1, 2):
        pass
    mw, m, v = w.clone().cuda(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lp = torch.empty(n, dtype=BF, device="cuda")
    rw, rm, rv = w.clone(), torch.zeros(n), torch.zeros(n)
    for step in (1, 2, 3):
        raw.adam_step(mw, lp, g.cuda(), m, v, 1e-2, 0.9, 0.99, 1e-8, 0.01, step)
        raw.adam_step(rw, None, g, rm, rv, 1e-2, 0.9, 0.99, 1e-8, 0.01, step)
    close(mw, rw, tol=1e-4)
    close(lp, rw, tol=1e-2)
    mw, vel = w.clone().cuda(), torch.zeros(n, device="cuda")
    rw, rvel = w.clone(), torch.zeros(n)
    for _ in range(3):
        raw.sgd_step(mw, lp, g.cuda(), vel, 0.1, 0.9)
        raw.sgd_step(rw, None, g, rvel, 0.1, 0.9)
    close(mw, rw, tol=1e-4)
    hyper = torch.tensor([0.5, 1.0, 1.0, 2.0], device="cuda")
    mw2 = w.clone().cuda()
    raw.sgd_step(mw2, None, g.cuda(), None, 0.0, 0.0, 1.0, hyper)
    close(mw2, w - 0.5 * 2.0 * g, tol=1e-4)


def test_functional_autograd_bridges_on_gpu():
    """ops/functional.py on bf16 CUDA tensors (tcgen05 GEMM, flash attention, layer norm and cross-entropy kernels
    behind torch.autograd) against the same expressions in fp32 torch on the CPU."""
    import torch.nn.functional as TF

    from tnn_b200.ops import functional as F

    torch.manual_seed(0)
    B, S, E, H, V = 2, 128, 128, 2, 1000
    mk = lambda *s, sc=1.0: (torch.randn(*s) * sc).to(BF).float()  # fp32 values that are exact in bf16
    x, delta, g1, b1 = mk(B, S, E), mk(B, S, E), mk(E) + 1, mk(E, sc=0.1)
    wqkv, bqkv, w1, bb1, wh = mk(3 * E, E, sc=0.08), mk(3 * E, sc=0.1), mk(4 * E, E, sc=0.08), mk(4 * E, sc=0.1), mk(V, 4 * E, sc=0.05)
    labels = torch.randint(0, V, (B, S))
    cpu = [t.clone().requires_grad_() for t in (x, delta, g1, b1, wqkv, bqkv, w1, bb1, wh)]
    gpu = [t.cuda().to(BF).requires_grad_() for t in (x, delta, g1, b1, wqkv, bqkv, w1, bb1, wh)]

    def ours(x, delta, g1, b1, wqkv, bqkv, w1, bb1, wh):
        h, s = F.add_layer_norm(x, delta, g1, b1, 1e-5)
        a = F.causal_self_attention(F.linear(h, wqkv, bqkv), H)
        return F.cross_entropy(F.linear(F.linear(a + s, w1, bb1, gelu=True), wh), labels.cuda())

    def theirs(x, delta, g1, b1, wqkv, bqkv, w1, bb1, wh):
        s = x + delta
        q, k, v = TF.linear(TF.layer_norm(s, (E,), g1, b1, 1e-5), wqkv, bqkv).split(E, dim=-1)
        hd = lambda t: t.reshape(B, S, H, E // H).transpose(1, 2)
        a = TF.scaled_dot_product_attention(hd(q), hd(k), hd(v), is_causal=True).transpose(1, 2).reshape(B, S, E)
        m = TF.linear(TF.gelu(TF.linear(a + s, w1, bb1), approximate="tanh"), wh)
        return TF.cross_entropy(m.reshape(-1, V), labels.reshape(-1))

    l1, l2 = ours(*gpu), theirs(*cpu)
    assert abs(l1.item() - l2.item()) < 3e-2 * abs(l2.item())
    l1.backward()
    l2.backward()
    _lib.check_status()
    for i, (a, b) in enumerate(zip(gpu, cpu)):
        assert a.grad is not None and a.grad.dtype == BF
        close(a.grad, b.grad, tol=6e-2, what=f"gradient {i}")


def test_example_torch_module_on_functional_ops_trains_on_gpu():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "torch_module_with_kernels.py")
    spec = importlib.util.spec_from_file_location("torch_module_with_kernels", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    first, last = mod.main("cuda", 40)
    _lib.check_status()
    assert last == last and last < 0.8 * first  # finite and decreasing with bf16 parameters
