"""The fp32 torch restatements in ops.raw (used as references for the kernels) against autograd."""
import pytest
import torch

from tnn_b200.ops import raw
from tnn_b200.ops.gemm import gemm, gelu_tanh_grad


def test_hash_uniform_range_and_rate():
    u = raw.hash_uniform(42, torch.arange(100000))
    assert 0 <= u.min() and u.max() < 1
    assert abs(u.mean().item() - 0.5) < 0.01
    assert abs((u >= 0.3).float().mean().item() - 0.7) < 0.01


def test_layernorm_matches_autograd():
    torch.manual_seed(0)
    x = torch.randn(17, 64, requires_grad=True)
    g = torch.randn(64, requires_grad=True)
    b = torch.randn(64, requires_grad=True)
    ref = torch.nn.functional.layer_norm(x, (64,), g, b, 1e-5)
    _, h, mean, rstd = raw.layernorm_fwd(x.detach(), None, g.detach(), b.detach(), 1e-5)
    assert torch.allclose(h, ref, atol=1e-5)
    dh = torch.randn(17, 64)
    ref.backward(dh)
    dg, db = torch.zeros(64), torch.zeros(64)
    dx, _ = raw.layernorm_bwd(dh, x.detach(), mean, rstd, g.detach(), None, False, 0.0, 0, dg, db)
    assert torch.allclose(dx, x.grad, atol=1e-4)
    assert torch.allclose(dg, g.grad, atol=1e-4) and torch.allclose(db, b.grad, atol=1e-4)


def test_attention_matches_autograd():
    torch.manual_seed(1)
    B, S, H, D = 2, 24, 2, 8
    qkv = torch.randn(B * S, 3 * H * D, requires_grad=True)
    q, k, v = (t.reshape(B, S, H, D).transpose(1, 2) for t in qkv.reshape(B * S, 3, H * D).unbind(1))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.3)
    ref = ref.transpose(1, 2).reshape(B * S, H * D)
    out, lse = raw.attn_fwd(qkv.detach(), B, S, H, D, True, 0.3)
    assert torch.allclose(out, ref, atol=1e-5)
    do = torch.randn_like(ref)
    ref.backward(do)
    d = raw.attn_bwd(qkv.detach(), out, do, lse, B, S, H, D, True, 0.3)
    assert torch.allclose(d, qkv.grad, atol=1e-4)


def test_softmax_ce_matches_autograd():
    torch.manual_seed(2)
    z = torch.randn(9, 13, requires_grad=True)
    y = torch.randint(0, 13, (9,))
    ref = torch.nn.functional.cross_entropy(z, y)
    ref.backward()
    loss, corr, grad = raw.softmax_ce(z.detach(), y, 13, 1.0 / 9, 1.0 / 9)
    assert torch.allclose(loss[0], ref, atol=1e-5)
    assert torch.allclose(grad, z.grad, atol=1e-5)
    assert int(corr) == int((z.argmax(1) == y).sum())


def test_gelu_grad_and_cpu_gemm_epilogues():
    x = torch.linspace(-4, 4, 101, requires_grad=True)
    torch.nn.functional.gelu(x, approximate="tanh").sum().backward()
    assert torch.allclose(gelu_tanh_grad(x.detach()), x.grad, atol=1e-5)
    a, b = torch.randn(5, 7), torch.randn(3, 7)
    out = gemm(a, b, bias=torch.ones(3), relu=True, out_dtype=torch.float32)
    assert torch.allclose(out, torch.relu(a @ b.t() + 1), atol=1e-5)
    acc = torch.ones(3, 7)
    gemm(torch.randn(11, 3), torch.randn(11, 7), a_t=True, b_t=True, out=acc, atomic=True)
    assert acc.shape == (3, 7)


def test_adam_matches_reference_formula():
    w = torch.tensor([1.0, -2.0])
    g = torch.tensor([0.5, 0.25])
    m, v = torch.zeros(2), torch.zeros(2)
    raw.adam_step(w, None, g, m, v, 0.1, 0.9, 0.999, 1e-8, 0.01, 1)
    mh, vh = g, g * g
    exp = torch.tensor([1.0, -2.0]) - 0.1 * mh / (vh.sqrt() + 1e-8) - 0.01 * 0.1 * torch.tensor([1.0, -2.0])
    assert torch.allclose(w, exp, atol=1e-6)


def test_named_ops_api():
    from tnn_b200.ops import tensor_ops as T

    a, b, c = torch.tensor([1.0, -2.0, 3.0]), torch.tensor([4.0, 5.0, -6.0]), torch.tensor([0.5, 0.5, 0.5])
    assert torch.equal(T.fmadd(a, b, c), a * b + c) and torch.equal(T.fnmadd(a, b, c), c - a * b) and torch.equal(T.fmsub(a, b, c), a * b - c)
    assert torch.equal(T.sub_mul_scalar(a, b, 2.0), (a - b) * 2) and torch.equal(T.mul_add_scalar(a, 2.0, 1.0), a * 2 + 1)
    y = c.clone()
    assert torch.equal(T.axpy(2.0, a, y), c + 2 * a) and y is not c
    assert float(T.dot_product(a, b)) == -24.0 and float(T.norm_squared(a)) == 14.0 and float(T.sum_squared_diff(a, 1.0)) == 13.0
    assert torch.equal(T.scalar_max(a, 0.0), torch.tensor([1.0, 0.0, 3.0])) and torch.equal(T.greater(a, b), torch.tensor([0.0, 0.0, 1.0]))
    x = torch.tensor([1, 256, 0x01020304], dtype=torch.int32)
    assert T.bswap(x).tolist() == [0x01000000, 0x00010000, 0x04030201] and torch.equal(T.bswap(T.bswap(x)), x)
    u = T.fill_random_uniform(torch.empty(1000), -1.0, 1.0, seed=3)
    assert -1.0 <= float(u.min()) and float(u.max()) <= 1.0 and torch.equal(u, T.fill_random_uniform(torch.empty(1000), -1.0, 1.0, seed=3))
    assert T.check_equals(a, a + 1e-4, tol=1e-3) and not T.check_equals(a, a + 1e-2, tol=1e-3)
    assert T.cast(a, torch.bfloat16).dtype == torch.bfloat16


def test_functional_autograd_bridges_match_torch():
    """ops/functional.py: the autograd Functions around the kernels (here their CPU references) against plain torch
    autograd on the same expressions - a GPT-2 style block written as an ordinary module trains through them."""
    import torch.nn.functional as TF

    from tnn_b200.ops import functional as F

    torch.manual_seed(0)
    B, S, E, H, V = 2, 8, 16, 2, 11
    x = torch.randn(B, S, E, requires_grad=True)
    delta = torch.randn(B, S, E, requires_grad=True)
    g1, b1 = torch.randn(E, requires_grad=True), torch.randn(E, requires_grad=True)
    wqkv, bqkv = (torch.randn(3 * E, E) * 0.2).requires_grad_(), torch.randn(3 * E, requires_grad=True)
    w1, bb1 = (torch.randn(4 * E, E) * 0.2).requires_grad_(), torch.randn(4 * E, requires_grad=True)
    wh = (torch.randn(V, E) * 0.2).requires_grad_()
    labels = torch.randint(0, V, (B, S))
    params = [x, delta, g1, b1, wqkv, bqkv, w1, bb1, wh]

    def ours():
        h, s = F.add_layer_norm(x, delta, g1, b1, 1e-5)
        a = F.causal_self_attention(F.linear(h, wqkv, bqkv), H)
        m = F.linear(F.linear(a + s, w1, bb1, gelu=True)[..., :E].contiguous(), wh)
        return F.cross_entropy(m, labels, return_corrects=True)

    def theirs():
        s = x + delta
        h = TF.layer_norm(s, (E,), g1, b1, 1e-5)
        q, k, v = TF.linear(h, wqkv, bqkv).split(E, dim=-1)
        hd = lambda t: t.reshape(B, S, H, E // H).transpose(1, 2)
        a = TF.scaled_dot_product_attention(hd(q), hd(k), hd(v), is_causal=True).transpose(1, 2).reshape(B, S, E)
        m = TF.linear(TF.gelu(TF.linear(a + s, w1, bb1), approximate="tanh")[..., :E], wh)
        return TF.cross_entropy(m.reshape(-1, V), labels.reshape(-1)), (m.argmax(-1) == labels).sum()

    (l1, c1), (l2, c2) = ours(), theirs()
    assert abs(float(l1) - float(l2)) < 1e-5 and int(c1) == int(c2)
    ga = torch.autograd.grad(l1, params)
    gb = torch.autograd.grad(l2, params)
    for a, b, p in zip(ga, gb, params):
        assert a.shape == p.shape and torch.allclose(a.float(), b, atol=2e-5, rtol=1e-4), (a - b).abs().max()
    # a scaled loss scales the gradients (the saved gradient of the cross-entropy is multiplied by the incoming one)
    l3, _ = ours()
    g3, = torch.autograd.grad(3.0 * l3, [wh])
    assert torch.allclose(g3, 3.0 * gb[-1], atol=1e-4)


def test_example_torch_module_on_functional_ops_trains():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "torch_module_with_kernels.py")
    spec = importlib.util.spec_from_file_location("torch_module_with_kernels", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    first, last = mod.main("cpu", 25)
    assert last < 0.6 * first


@pytest.mark.parametrize("h,wd,c,o,k,s,p", [(16, 16, 4, 6, 3, 2, 1), (15, 17, 4, 6, 3, 2, 1), (16, 16, 4, 6, 1, 2, 0),
                                            (14, 14, 3, 5, 7, 2, 3), (12, 12, 2, 3, 5, 3, 2), (9, 9, 2, 3, 3, 2, 0)])
def test_strided_dgrad_parity_classes(h, wd, c, o, k, s, p):
    """The decomposition the GPU path uses for the data gradient of a strided convolution: every parity class of input
    pixels is a stride-1 correlation of ``dy`` with the sub-filter ``_parity_classes`` names. Restated here with
    plain torch convolutions (same taps, same padding) and compared with ``conv2d_input``."""
    import torch.nn.functional as F
    from tnn_b200.ops.conv import _parity_classes
    torch.manual_seed(0)
    oh, ow = (h + 2 * p - k) // s + 1, (wd + 2 * p - k) // s + 1
    dy, w = torch.randn(2, oh, ow, o), torch.randn(o, k, k, c)
    ref = torch.nn.grad.conv2d_input((2, c, h, wd), w.permute(0, 3, 1, 2), dy.permute(0, 3, 1, 2), s, p).permute(0, 2, 3, 1)
    dx = torch.zeros(2, h, wd, c)
    for a, hc, khs, phc in _parity_classes(h, k, s, p):
        for b, wc, kws, pwc in _parity_classes(wd, k, s, p):
            if not khs or not kws or hc <= 0 or wc <= 0:
                continue
            # the same strided slice + flip the GPU path takes (no index tensors)
            w_sub = w[:, khs[-1]::s, kws[-1]::s].flip(1, 2)
            assert torch.equal(w_sub, w[:, khs][:, :, kws])
            pt, pl = max(phc, 0), max(pwc, 0)
            pb = max(0, hc - 1 + len(khs) - 1 - phc - (oh - 1))
            pr = max(0, wc - 1 + len(kws) - 1 - pwc - (ow - 1))
            d = F.pad(dy.permute(0, 3, 1, 2), (pl, pr, pt, pb))[:, :, pt - phc:, pl - pwc:]
            y = F.conv2d(d, w_sub.permute(3, 0, 1, 2))[:, :, :hc, :wc]   # filter [C, O, th, tw]
            dx[:, a::s, b::s, :] = y.permute(0, 2, 3, 1)
    assert torch.allclose(dx, ref, atol=1e-4, rtol=1e-4)
