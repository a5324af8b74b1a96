"""Graph builder / executor on CPU: fused segments vs layer-by-layer execution, autograd parity,
fan-out accumulation, micro-batch contexts and TNNG round trips."""
import torch

from tnn_b200.io import tnng
from tnn_b200.models import zoo
from tnn_b200.nn.graph import Graph
from tnn_b200.nn.layers import Dense, ReLU
from tnn_b200.nn.loss import CrossEntropyLoss


def tiny_gpt(drop=0.0):
    return zoo.gpt2(64, 1, 2, "tiny", seq_len=16, vocab=50, drop=drop)


def run(g, ids, labels):
    out = g.forward({"input": ids})["output"]
    loss, grad = CrossEntropyLoss().compute(out, labels)
    g.backward({"output": grad})
    return loss, g.grads_flat.clone()


def test_fused_gpt_chain_equals_unfused():
    torch.manual_seed(0)
    ids = torch.randint(0, 50, (3, 16))
    labels = torch.randint(0, 50, (3, 16))
    a = tiny_gpt().compile(seed=1, fuse=True)
    b = tiny_gpt().compile(seed=1, fuse=False)
    assert any(type(s).__name__ == "_GPTChain" for s in a.segments)
    assert any(type(s).__name__ == "_EmbedSegment" for s in a.segments)
    assert all(type(s).__name__ == "_EdgeSegment" for s in b.segments)
    la, ga = run(a, ids, labels)
    lb, gb = run(b, ids, labels)
    assert torch.allclose(la, lb, atol=1e-5)
    assert torch.allclose(ga, gb, atol=1e-4, rtol=1e-3)


def test_recompute_qkv_gives_the_same_gradients():
    """Dropping the saved q/k/v projection and computing it again in the backward pass (what the reference's
    attention block always does) must not change loss or gradients, fused chain or layer by layer."""
    torch.manual_seed(0)
    ids = torch.randint(0, 50, (3, 16))
    labels = torch.randint(0, 50, (3, 16))
    for fuse in (True, False):
        a = tiny_gpt().compile(seed=1, fuse=fuse)
        b = tiny_gpt().compile(seed=1, fuse=fuse)
        assert b.set_recompute_qkv(True) >= 1
        la, ga = run(a, ids, labels)
        lb, gb = run(b, ids, labels)
        assert torch.allclose(la, lb, atol=1e-6) and torch.allclose(ga, gb, atol=1e-6)


def test_gpt_matches_torch_autograd():
    torch.manual_seed(1)
    g = tiny_gpt().compile(seed=2)
    ids = torch.randint(0, 50, (2, 16))
    labels = torch.randint(0, 50, (2, 16))
    loss, grads = run(g, ids, labels)
    # re-express the model with torch ops on leaf copies of the same parameters
    L = {l.name: l for l in g.layers()}
    P = {}

    def leaf(t):
        p = t.detach().clone().requires_grad_(True)
        P[id(t)] = p
        return p

    x = leaf(L["token_embed"].params[0])[ids] + leaf(L["pos_embed"].params[0])
    for i in range(2):
        n = f"tiny_block_{i}"
        ln1, at, ln2, f1, f2 = L[n + "_ln_1"], L[n + "_attn"], L[n + "_ln_2"], L[n + "_mlp_fc1"], L[n + "_mlp_fc2"]
        h = torch.nn.functional.layer_norm(x, (64,), leaf(ln1.params[0]), leaf(ln1.params[1]), 1e-5)
        qkv = h @ leaf(at.params[0]).t() + leaf(at.params[1])
        q, k, v = (t.reshape(2, 16, 1, 64).transpose(1, 2) for t in qkv.split(64, -1))
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0)
        x = x + a.transpose(1, 2).reshape(2, 16, 64) @ leaf(at.params[2]).t() + leaf(at.params[3])
        h = torch.nn.functional.layer_norm(x, (64,), leaf(ln2.params[0]), leaf(ln2.params[1]), 1e-5)
        h = torch.nn.functional.gelu(h @ leaf(f1.params[0]).t() + leaf(f1.params[1]), approximate="tanh")
        x = x + h @ leaf(f2.params[0]).t() + leaf(f2.params[1])
    x = torch.nn.functional.layer_norm(x, (64,), leaf(L["ln_f"].params[0]), leaf(L["ln_f"].params[1]), 1e-5)
    logits = x @ leaf(L["head"].params[0]).t() + leaf(L["head"].params[1])
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 50), labels.reshape(-1))
    ref.backward()
    assert torch.allclose(loss[0], ref, atol=1e-5)
    for l in g.layers():
        for p, gr in zip(l.params, l.grads):
            assert torch.allclose(gr, P[id(p)].grad, atol=2e-4, rtol=1e-3), l.name


def test_fanout_accumulates_and_contexts_are_per_microbatch():
    g = Graph()
    x = g.input("input")
    h = Dense(4, 4, name="a")(x)
    y = ReLU(name="r")(h) + h
    y.set_uid("output")
    g.set_output(y)
    g.compile(seed=3)
    g.input_requires_grad = True
    x0, x1 = torch.randn(2, 4), torch.randn(2, 4)
    o0 = g.forward({"input": x0}, pid=0)["output"]
    o1 = g.forward({"input": x1}, pid=1)["output"]
    gi1 = g.backward({"output": torch.ones_like(o1)}, pid=1)["input"]
    gi0 = g.backward({"output": torch.ones_like(o0)}, pid=0)["input"]
    w = g.layers()[0].params[0]
    for xi, gi in ((x0, gi0), (x1, gi1)):
        hpre = xi @ w.t() + g.layers()[0].params[1]
        expect = ((hpre > 0).float() + 1) @ w
        assert torch.allclose(gi, expect, atol=1e-5)


def test_tnng_round_trip_and_reference_layout(tmp_path):
    g = zoo.create("cifar10_resnet9")
    g.compile(seed=4)
    path = str(tmp_path / "m.tnng")
    g.save_state(path)
    raw_bytes = open(path, "rb").read()
    assert raw_bytes[:4] == b"TNNG" and int.from_bytes(raw_bytes[4:8], "little") == 2
    st = tnng.read_file(path)
    assert st["nodes"][0] == "input" and "output" in st["nodes"]
    assert '"type":"conv2d"' in st["layers"][0] and '"unsigned long"' in st["layers"][0]
    g2 = Graph.load_state(path)
    x = torch.randn(2, 32, 32, 3)
    g.eval()
    g2.eval()
    assert torch.allclose(g(x), g2(x), atol=1e-5)
    # batchnorm keeps the reference's four tensors per layer
    bn = [i for i, s in enumerate(st["layers"]) if '"type":"batchnorm"' in s][0]
    assert len(st["params"][bn]) == 4


def test_attention_block_checkpoint_has_eight_tensors():
    g = tiny_gpt().compile(seed=5)
    st = g.state()
    idx = [i for i, s in enumerate(st["layers"]) if "flash_attention_block" in s][0]
    shapes = [tuple(t.shape) for t in st["params"][idx]]
    assert shapes == [(64, 64), (64,), (64, 64), (64,), (64, 64), (64,), (64, 64), (64,)]
    g2 = Graph.from_state(tnng.parse(tnng.serialize(st)))
    ids = torch.randint(0, 50, (1, 16))
    g.eval(); g2.eval()
    assert torch.allclose(g(ids), g2(ids), atol=1e-5)


def test_memory_report_counts_params_and_saved_tensors():
    from tnn_b200.models import zoo

    g = zoo.create("cifar10_resnet9").compile(device="cpu", seed=1)
    g.train()
    g(torch.randn(2, 32, 32, 3))
    rows = g.memory_report()
    assert len(rows) == len(g.segments)
    assert sum(r[1] for r in rows) == g.params_flat.numel() * g.params_flat.element_size() or \
        sum(r[1] for r in rows) <= g.params_flat.numel() * g.params_flat.element_size()  # slab has alignment padding
    assert sum(r[1] for r in rows) >= g.num_parameters() * g.params_flat.element_size()
    assert sum(r[2] for r in rows) > 0
    assert "total" in g.format_memory_report()


def test_batchnorm_without_affine_still_saves_four_tensors(tmp_path):
    """The reference lists gamma, beta, running_mean, running_var for every batch norm, affine or not
    (include/nn/layers_impl/batchnorm_layer.hpp:51-81): a file of an affine=false layer must carry all four and load
    back, and the untrained gamma / beta must not influence the output."""
    from tnn_b200.models import zoo
    from tnn_b200.nn.layers import BatchNorm

    def build():
        b = zoo._start((1, 8, 8, 3))
        b.conv(4, 3, 1, 1, False, "c1")
        b.apply(BatchNorm(4, 1e-5, 0.1, False, False, name="bn_plain"))
        return zoo._finish(b.flatten().dense(5, True, "fc"))

    g = build().compile(device="cpu", seed=3)
    bn = [l for l in g.layers() if l.name == "bn_plain"][0]
    assert [s.name for s in bn.param_specs()] == ["gamma", "beta", "running_mean", "running_var"]
    assert [s.trainable for s in bn.param_specs()] == [False, False, False, False]
    x = torch.randn(6, 8, 8, 3)
    g.set_training(True)
    y = g.forward({"input": x})["output"]
    bn.params[0].fill_(7.0)   # gamma of a non-affine layer is carried along, not used
    y2 = g.forward({"input": x})["output"]
    assert torch.allclose(y, y2)
    path = str(tmp_path / "bn.tnng")
    g.save_state(path)
    g2 = Graph.load_state(path, device="cpu")
    bn2 = [l for l in g2.layers() if l.name == "bn_plain"][0]
    assert len(bn2.params) == 4 and not bn2.affine
    assert torch.allclose(bn2.params[0], bn.params[0]) and torch.allclose(bn2.params[3], bn.params[3])


def test_bottleneck_add_fusions_match_edge_by_edge():
    """The executor's two residual-block fusions (closing add inside the last batch norm's segment, gradient of the
    block input summed by the first convolution's data-gradient pass) give what the plain edge-by-edge run gives."""
    from tnn_b200.models.zoo import _start, _finish, bottleneck_block

    def build():
        b = _start((1, 8, 8, 16))
        b = bottleneck_block(b, 8, 32, 1, "b1")
        b = bottleneck_block(b, 8, 32, 1, "b2")
        b = bottleneck_block(b, 16, 64, 2, "b3")
        return _finish(b)

    torch.manual_seed(0)
    gf = build().compile(device="cpu", seed=4)
    gu = build().compile(device="cpu", seed=4, fuse=False)
    gf.input_requires_grad = gu.input_requires_grad = True
    assert [type(s).__name__ for s in gf.segments].count("_BnAddSegment") == 3
    assert all(type(s).__name__ == "_EdgeSegment" for s in gu.segments)
    x, dy = torch.randn(4, 8, 8, 16), torch.randn(4, 4, 4, 64)
    of, ou = gf.forward({"input": x})["output"], gu.forward({"input": x})["output"]
    assert torch.allclose(of, ou, atol=1e-6)
    gi, gj = gf.backward({"output": dy})["input"], gu.backward({"output": dy})["input"]
    assert torch.allclose(gi, gj, rtol=1e-5, atol=1e-5 * float(gj.abs().max()))
    a = torch.cat([g.reshape(-1) for l in gf.layers() for g in l.grads if g is not None])
    b = torch.cat([g.reshape(-1) for l in gu.layers() for g in l.grads if g is not None])
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(b.abs().max()))
    # and against autograd on the same arithmetic: finite difference of sum(out * dy) along a random direction
    d = torch.randn_like(x)
    eps = 1e-3
    fp = (gu.forward({"input": x + eps * d})["output"] * dy).sum()
    fm = (gu.forward({"input": x - eps * d})["output"] * dy).sum()
    fd = float((fp - fm) / (2 * eps))
    an = float((gi * d).sum())
    assert abs(fd - an) <= 6e-2 * max(abs(fd), abs(an)) + 1e-3, (fd, an)  # ReLU kinks inside the step
