"""Convolution / batch-norm / pooling kernels and a CNN training step against the fp32 CPU path."""
import pytest
import torch

from tnn_b200.models import zoo
from tnn_b200.nn.loss import CrossEntropyLoss
from tnn_b200.ops import _lib, raw

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape) * scale).to(BF)


def close(got, ref, tol=2e-2, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"{what} rel err {err / scale:.4g}"
    # and element by element: 3 % of the element plus half of that tolerance times the largest value
    bad = (got - ref).abs() > (3e-2 * ref.abs() + 0.5 * tol * scale)
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} elements outside the per-element tolerance"


@pytest.mark.parametrize("n,h,c,o,k,s,p", [(2, 16, 64, 64, 3, 1, 1), (2, 15, 32, 48, 3, 2, 1), (3, 14, 64, 128, 1, 1, 0),
                                           (2, 14, 64, 128, 1, 2, 0), (2, 20, 3, 16, 7, 2, 3), (1, 9, 8, 24, 5, 1, 0),
                                           (2, 8, 16, 16, 3, 1, 1),
                                           # implicit-GEMM routes (channel counts multiple of 64): odd batch and spatial sizes,
                                           # strided 3x3, 7x7 maps, more than one column block
                                           (3, 28, 64, 64, 3, 1, 1), (4, 14, 128, 256, 3, 2, 1), (3, 7, 256, 64, 3, 1, 1),
                                           # strided layers, odd sizes: the data gradient runs as one launch per parity class
                                           (3, 15, 64, 128, 3, 2, 1), (2, 13, 128, 64, 1, 2, 0), (2, 18, 64, 64, 5, 3, 2),
                                           # 64 -> 64 channels, stride 1: the kernels that load one input window per tile
                                           (2, 20, 64, 64, 3, 1, 0), (2, 17, 64, 64, 2, 1, 0), (5, 56, 64, 64, 3, 1, 1),
                                           (5, 9, 64, 320, 3, 1, 1), (2, 12, 192, 128, 5, 1, 2)])
def test_conv2d(n, h, c, o, k, s, p):
    torch.manual_seed(0)
    x, w, b = rnd(n, h, h, c), rnd(o, k, k, c, scale=0.2), rnd(o)
    y = raw.conv2d_fwd(x.cuda(), w.cuda(), b.cuda(), (s, s), (p, p))
    ry = raw.conv2d_fwd(x, w, b, (s, s), (p, p))
    close(y, ry, what="fwd")
    dy = rnd(*ry.shape)
    close(raw.conv2d_dgrad(dy.cuda(), w.cuda(), x.shape, (s, s), (p, p)), raw.conv2d_dgrad(dy, w, x.shape, (s, s), (p, p)),
          what="dgrad")
    dw, rdw = torch.ones(w.shape, device="cuda"), torch.ones(w.shape)
    raw.conv2d_wgrad(x.cuda(), dy.cuda(), dw, (s, s), (p, p))
    raw.conv2d_wgrad(x, dy, rdw, (s, s), (p, p))
    close(dw, rdw, what="wgrad")
    _lib.check_status()


@pytest.mark.parametrize("shape", [(4, 8, 8, 64), (2, 7, 7, 256), (3, 5, 5, 8), (64, 512)])
@pytest.mark.parametrize("relu,affine", [(True, True), (False, True), (False, False)])
def test_batchnorm(shape, relu, affine):
    torch.manual_seed(1)
    C = shape[-1]
    x = rnd(*shape) + 0.5
    g, b = (rnd(C) + 1, rnd(C)) if affine else (None, None)
    rm, rv = torch.zeros(C), torch.ones(C)
    crm, crv = rm.cuda(), rv.cuda()
    y, mean, rstd = raw.batchnorm_fwd_train(x.cuda(), None if g is None else g.cuda(), None if b is None else b.cuda(), crm, crv,
                                            1e-5, 0.1, relu)
    ry, rmean, rrstd = raw.batchnorm_fwd_train(x, g, b, rm, rv, 1e-5, 0.1, relu)
    close(y, ry, what="y")
    close(mean, rmean, tol=1e-3)
    close(rstd, rrstd, tol=1e-2)
    close(crm, rm, tol=1e-3)
    close(crv, rv, tol=1e-2)
    dy = rnd(*shape)
    dg, db = (torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")) if affine else (None, None)
    rdg, rdb = (torch.zeros(C), torch.zeros(C)) if affine else (None, None)
    dx = raw.batchnorm_bwd(dy.cuda(), x.cuda(), y, mean, rstd, None if g is None else g.cuda(), dg, db, relu)
    rdx = raw.batchnorm_bwd(dy, x, ry, rmean, rrstd, g, rdg, rdb, relu)
    close(dx, rdx, tol=4e-2, what="dx")
    if affine:
        close(dg, rdg, tol=3e-2)
        close(db, rdb, tol=3e-2)
    if relu:
        # the same backward with the ReLU mask recomputed from x (beta given, y never read) must agree (up to the order of the atomic partial sums)
        dg2, db2 = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        dx2 = raw.batchnorm_bwd(dy.cuda(), x.cuda(), None, mean, rstd, g.cuda(), dg2, db2, relu, beta=b.cuda())
        close(dx2, dx, tol=1e-3, what="dx with recomputed mask")  # one flipped mask element would be an O(1) difference
        close(dg2, dg, tol=1e-4)
        close(db2, db, tol=1e-4)
    yi = raw.batchnorm_infer(x.cuda(), None if g is None else g.cuda(), None if b is None else b.cuda(), crm, crv, 1e-5, relu)
    close(yi, raw.batchnorm_infer(x, g, b, rm, rv, 1e-5, relu), what="infer")


@pytest.mark.parametrize("shape", [(4, 8, 8, 64), (3, 5, 5, 8), (37, 7, 7, 256)])
def test_batchnorm_with_closing_residual_add(shape):
    """y = relu(bn(x) + shortcut) in the batch norm's own pass, training and inference, and a bottleneck-style
    residual block (main path ending in a batch norm without ReLU) through the layer API against the CPU path."""
    torch.manual_seed(2)
    C = shape[-1]
    x, res = rnd(*shape) + 0.3, rnd(*shape)
    g, b = rnd(C) + 1, rnd(C)
    rm, rv = torch.zeros(C), torch.ones(C)
    crm, crv = rm.cuda(), rv.cuda()
    y, mean, rstd = raw.batchnorm_fwd_train(x.cuda(), g.cuda(), b.cuda(), crm, crv, 1e-5, 0.1, True, resid=res.cuda())
    ry, rmean, rrstd = raw.batchnorm_fwd_train(x, g, b, rm, rv, 1e-5, 0.1, True, resid=res)
    _lib.check_status()
    close(y, ry, what="y")
    assert float(y.min()) >= 0.0
    close(mean, rmean, tol=1e-3)
    close(crv, rv, tol=1e-2)
    close(raw.batchnorm_infer(x.cuda(), g.cuda(), b.cuda(), crm, crv, 1e-5, False, resid=res.cuda()),
          raw.batchnorm_infer(x, g, b, rm, rv, 1e-5, False, resid=res), what="infer")


def test_residual_block_with_fused_closing_add():
    """A bottleneck-style block (main path ending in a batch norm without ReLU): the closing add + ReLU done inside
    that batch norm gives the same output, input gradient and parameter gradients as the separate add kernel (both in
    bf16 on the GPU), and the output agrees with the fp32 CPU path."""
    from tnn_b200.nn import layers as L
    from tnn_b200.nn.blocks import ResidualBlock, Sequential
    from tnn_b200.nn.graph import Graph

    def build(fused=True, shortcut=False):
        g = Graph()
        main = Sequential([L.Conv2D(64, 64, 3, 3, 1, 1, 1, 1, name="c1"), L.BatchNorm(64, use_relu=True, name="b1"),
                           L.Conv2D(64, 128 if shortcut else 64, 1, 1, 1, 1, 0, 0, name="c2"),
                           L.BatchNorm(128 if shortcut else 64, name="b2")], name="main")
        sc = Sequential([L.Conv2D(64, 128, 1, 1, 1, 1, 0, 0, name="sc"), L.BatchNorm(128, name="sb")], name="short") if shortcut else None
        blk = ResidualBlock(main, sc, "relu", name="block")
        if not fused:
            blk._closing_add_in_batchnorm = lambda x: False
        out = blk(g.input("input"))
        out.set_uid("output")
        g.set_output(out)
        g.input_requires_grad = True
        return g

    torch.manual_seed(3)
    x, dy = rnd(8, 12, 12, 64), rnd(8, 12, 12, 64)
    for shortcut in (False, True):
        dyy = torch.cat([dy, dy], -1) if shortcut else dy
        a = build(True, shortcut).compile(device="cuda", seed=0)
        b = build(False, shortcut).compile(device="cuda", seed=0)
        assert torch.equal(a.master_flat, b.master_flat)
        ya, yb = a.forward({"input": x.cuda()})["output"], b.forward({"input": x.cuda()})["output"]
        close(ya, yb, tol=1e-3, what="output, fused vs separate add")
        da, db = a.backward({"output": dyy.cuda()})["input"], b.backward({"output": dyy.cuda()})["input"]
        _lib.check_status()
        close(da, db, tol=5e-3, what="input gradient")
        close(a.grads_flat, b.grads_flat, tol=5e-3, what="parameter gradients")
        if not shortcut:
            cpu = build(True).compile(device="cpu", seed=0)
            for lc, lg in zip(cpu.layers(), a.layers()):  # bf16-rounded weights on both sides
                for pc, pg in zip(lc.params, lg.params):
                    pc.copy_(pg.float().cpu())
            close(ya, cpu.forward({"input": x.float()})["output"], tol=4e-2, what="output vs fp32 CPU")


@pytest.mark.parametrize("mode", ["max", "avg"])
@pytest.mark.parametrize("h,k,s,p", [(8, 2, 2, 0), (9, 3, 2, 1), (7, 7, 1, 0), (6, 3, 3, 0)])
def test_pool(mode, h, k, s, p):
    torch.manual_seed(2)
    x = rnd(2, h, h, 16)
    y, idx = raw.pool2d_fwd(x.cuda(), mode, (k, k), (s, s), (p, p))
    ry, ridx = raw.pool2d_fwd(x, mode, (k, k), (s, s), (p, p))
    close(y, ry, tol=1e-2)
    dy = rnd(*ry.shape)
    dx = raw.pool2d_bwd(dy.cuda(), idx, x.shape, mode, (k, k), (s, s), (p, p))
    rdx = raw.pool2d_bwd(dy, ridx, x.shape, mode, (k, k), (s, s), (p, p))
    close(dx, rdx, tol=2e-2)


def test_resnet9_step_matches_cpu():
    torch.manual_seed(3)
    x = torch.randn(4, 32, 32, 3)
    labels = torch.randint(0, 10, (4,))
    gc = zoo.create("cifar10_resnet9").compile(device="cpu", seed=9)
    gg = zoo.create("cifar10_resnet9").compile(device="cuda", seed=9)
    for lc, lg in zip(gc.layers(), gg.layers()):  # bf16-rounded weights on both sides (slab layouts differ by dtype)
        for pc, pg in zip(lc.params, lg.params):
            pc.copy_(pg.float().cpu())
    oc = gc.forward({"input": x})["output"]
    og = gg.forward({"input": x.cuda()})["output"]
    _lib.check_status()
    assert (og.float().cpu() - oc).abs().max() < 0.2 * oc.abs().max() + 0.05
    lc, gradc = CrossEntropyLoss().compute(oc, labels)
    lg, gradg = CrossEntropyLoss().compute(og, labels.cuda())
    gc.backward({"output": gradc})
    gg.backward({"output": gradg})
    _lib.check_status()
    # per tensor: the flat buffers are padded differently for fp32 and bf16 parameters
    a = torch.cat([g.reshape(-1).float() for l in gc.layers() for g in l.grads if g is not None])
    b = torch.cat([g.reshape(-1).float().cpu() for l in gg.layers() for g in l.grads if g is not None])
    cos = torch.nn.functional.cosine_similarity(a, b, dim=0)
    assert cos > 0.95, float(cos)  # bf16 batch-norm statistics over a batch of 4 are noisy


def _bottleneck_graph():
    from tnn_b200.models.zoo import _start, _finish, bottleneck_block
    b = _start((1, 16, 16, 64))
    b = bottleneck_block(b, 32, 128, 1, "b1")   # projection shortcut (channels change)
    b = bottleneck_block(b, 32, 128, 1, "b2")   # identity shortcut
    b = bottleneck_block(b, 64, 256, 2, "b3")   # strided projection shortcut
    return _finish(b)


def test_bottleneck_blocks_fused_add_paths():
    """Graph-level fusions of a bottleneck stack: the block's closing add runs inside the last batch norm's pass
    (y = relu(bn(x)) + shortcut) and the gradient of the block input is summed in the first convolution's data
    gradient GEMM. Compared with the same graph run edge by edge on the GPU and with the fp32 CPU path."""
    torch.manual_seed(5)
    x = torch.randn(8, 16, 16, 64)
    dy = torch.randn(8, 8, 8, 256) * 0.1
    gf = _bottleneck_graph().compile(device="cuda", seed=4)
    gu = _bottleneck_graph().compile(device="cuda", seed=4, fuse=False)
    gc = _bottleneck_graph().compile(device="cpu", seed=4)
    for g in (gf, gu, gc):
        g.input_requires_grad = True
    names = [type(s).__name__ for s in gf.segments]
    assert names.count("_BnAddSegment") == 3 and "_BnAddSegment" not in [type(s).__name__ for s in gu.segments]
    for lf, lu, lc in zip(gf.layers(), gu.layers(), gc.layers()):
        for pf, pu, pc in zip(lf.params, lu.params, lc.params):
            pu.copy_(pf)
            pc.copy_(pf.float().cpu())
    of = gf.forward({"input": x.cuda()})["output"]
    ou = gu.forward({"input": x.cuda()})["output"]
    oc = gc.forward({"input": x})["output"]
    _lib.check_status()
    # same kernels, same rounding points: the fused add sums the same two bf16 tensors
    assert torch.equal(of, ou)
    close(of, oc, tol=3e-2, what="bottleneck forward")
    gin_f = gf.backward({"output": dy.cuda().bfloat16()})["input"]
    gin_u = gu.backward({"output": dy.cuda().bfloat16()})["input"]
    gin_c = gc.backward({"output": dy.bfloat16().float()})["input"]
    _lib.check_status()
    # the fused gradient sum rounds once (fp32 sum in the GEMM epilogue) where the separate add rounds twice
    close(gin_f, gin_u, tol=2e-2, what="input gradient, fused vs edge by edge")
    # against fp32 only in direction: nine bf16 batch norms and their ReLU masks lie between the two ends
    cos_in = torch.nn.functional.cosine_similarity(gin_f.float().cpu().reshape(-1), gin_c.reshape(-1), dim=0)
    assert cos_in > 0.95, float(cos_in)
    a = torch.cat([g.reshape(-1).float().cpu() for l in gf.layers() for g in l.grads if g is not None])
    b = torch.cat([g.reshape(-1).float().cpu() for l in gu.layers() for g in l.grads if g is not None])
    c = torch.cat([g.reshape(-1).float() for l in gc.layers() for g in l.grads if g is not None])
    assert torch.nn.functional.cosine_similarity(a, b, dim=0) > 0.999
    assert torch.nn.functional.cosine_similarity(a, c, dim=0) > 0.95
