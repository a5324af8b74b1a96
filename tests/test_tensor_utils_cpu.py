"""Tensor utilities (pad / unpad / crop / split / layout conversions / patch matrices) against plain indexing."""
import pytest
import torch

from tnn_b200.ops import tensor_utils as tu


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_pad_unpad_crop_round_trip(layout):
    torch.manual_seed(0)
    x = torch.randn(2, 5, 6, 3) if layout == "nhwc" else torch.randn(2, 3, 5, 6)
    p = tu.pad(x, 2, 1, value=-7.0, layout=layout)
    dh, dw = (1, 2) if layout == "nhwc" else (2, 3)
    assert p.shape[dh] == 5 + 4 and p.shape[dw] == 6 + 2
    assert float(p.select(dh, 0).max()) == -7.0 and float(p.select(dw, 0).max()) == -7.0
    assert torch.equal(tu.unpad(p, 2, 1, layout=layout), x)
    c = tu.crop(x, 1, 2, 3, 4, layout=layout)    # both ends inclusive
    ref = x[:, 1:4, 2:5, :] if layout == "nhwc" else x[:, :, 1:4, 2:5]
    assert torch.equal(c, ref)
    out = torch.empty_like(ref)
    assert tu.crop(x, 1, 2, 3, 4, layout=layout, out=out) is out and torch.equal(out, ref)
    with pytest.raises(ValueError):
        tu.crop(x, 0, 0, 5, 2, layout=layout)
    with pytest.raises(ValueError):
        tu.pad(x[0], 1, 1)


def test_split_and_slice_batch():
    x = torch.arange(7 * 2).reshape(7, 2)
    parts = tu.split(x, 3)
    assert [p.shape[0] for p in parts] == [3, 2, 2] and torch.equal(torch.cat(parts), x)
    assert torch.equal(tu.slice_batch(x, 2, 5), x[2:5])
    for bad in (0, 8):
        with pytest.raises(ValueError):
            tu.split(x, bad)


def test_layout_conversions():
    x = torch.randn(2, 3, 4, 5)
    assert torch.equal(tu.cnhw_to_nchw(tu.nchw_to_cnhw(x)), x)
    assert tu.nchw_to_cnhw(x).shape == (3, 2, 4, 5) and tu.nchw_to_cnhw(x).is_contiguous()
    assert torch.equal(tu.nhwc_to_nchw(tu.nchw_to_nhwc(x)), x)
    m = torch.randn(4, 7)
    assert torch.equal(tu.transpose_2d(m), m.t())


@pytest.mark.parametrize("k,s,p", [((3, 3), (1, 1), (1, 1)), ((3, 2), (2, 1), (0, 1)), ((1, 1), (2, 2), (0, 0))])
def test_im2col_is_the_convolution_and_col2im_its_adjoint(k, s, p):
    torch.manual_seed(1)
    x = torch.randn(2, 7, 8, 3)
    w = torch.randn(4, k[0], k[1], 3)              # KRSC
    cols = tu.im2col(x, k, s, p)
    y = (cols @ w.reshape(4, -1).t())
    ref = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), stride=s, padding=p)
    assert torch.allclose(y.reshape(2, ref.shape[2], ref.shape[3], 4).permute(0, 3, 1, 2), ref, atol=1e-4)
    # <im2col(x), c> == <x, col2im(c)>
    c = torch.randn_like(cols)
    back = tu.col2im(c, x.shape, k, s, p)
    assert abs(float((cols * c).sum()) - float((x * back).sum())) < 1e-2
    assert torch.allclose(tu.im2col(x.permute(0, 3, 1, 2), k, s, p, layout="nchw"), cols)


def test_fills_with_seed_are_reproducible():
    a, b = torch.empty(100), torch.empty(100)
    tu.fill_normal(a, 1.0, 2.0, seed=3)
    tu.fill_normal(b, 1.0, 2.0, seed=3)
    assert torch.equal(a, b) and abs(float(a.mean()) - 1.0) < 1.0
    tu.fill_uniform(a, -1.0, 1.0, seed=4)
    assert float(a.min()) >= -1.0 and float(a.max()) <= 1.0
    assert tu.check_equals(tu.fill(b, 2.5), torch.full((100,), 2.5))
