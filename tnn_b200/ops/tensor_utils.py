"""Tensor utilities of the reference's ``tensor_ops.hpp`` by name: fills, spatial pad / unpad / crop, batch slicing
and splitting, 2-D transpose, layout conversions and the patch-matrix pair ``im2col`` / ``col2im``
(include/tensor/tensor_ops.hpp:68-620).

The reference's legacy convolution path works on NCHW tensors and builds its patch matrices on the CPU or with SIMT
kernels; here activations are NHWC (channels innermost, what the implicit-GEMM kernels read), so every function
takes a ``layout`` argument: ``"nhwc"`` (default) or ``"nchw"`` for data that comes from or goes to the reference's
layout. Each result is a new contiguous tensor on the input's device; ``out=`` writes into a caller-owned tensor of
the right shape and dtype instead, like the reference's ``(input, result, ...)`` signatures.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

_LAYOUTS = ("nhwc", "nchw")


def _hw_dims(t: torch.Tensor, layout: str) -> Tuple[int, int]:
    if t.dim() != 4:
        raise ValueError("expected a 4-dimensional tensor")
    if layout not in _LAYOUTS:
        raise ValueError(f"layout must be one of {_LAYOUTS}")
    return (1, 2) if layout == "nhwc" else (2, 3)


def _emit(r: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
    if out is None:
        return r.contiguous()
    if tuple(out.shape) != tuple(r.shape) or out.dtype != r.dtype or out.device != r.device:
        raise ValueError(f"result tensor must be {tuple(r.shape)} {r.dtype} on {r.device}")
    out.copy_(r)
    return out


# ------------------------------------------------------------------------------------ fills
def fill(t: torch.Tensor, value: float) -> torch.Tensor:
    return t.fill_(value)


def fill_normal(t: torch.Tensor, mean: float, stddev: float, seed: Optional[int] = None) -> torch.Tensor:
    """Normal fill; with a seed the values do not depend on the device (drawn on the host in fp32)."""
    if seed is None:
        return t.normal_(mean, stddev)
    g = torch.Generator().manual_seed(int(seed))
    return t.copy_(torch.empty(t.shape, dtype=torch.float32).normal_(mean, stddev, generator=g))


def fill_uniform(t: torch.Tensor, low: float, high: float, seed: Optional[int] = None) -> torch.Tensor:
    if seed is None:
        return t.uniform_(low, high)
    g = torch.Generator().manual_seed(int(seed))
    return t.copy_(torch.empty(t.shape, dtype=torch.float32).uniform_(low, high, generator=g))


# -------------------------------------------------------------------------- spatial pad / crop
def pad(x: torch.Tensor, pad_h: int, pad_w: int, value: float = 0.0, layout: str = "nhwc",
        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``pad_h`` rows above and below, ``pad_w`` columns left and right, filled with ``value``."""
    dh, dw = _hw_dims(x, layout)
    shape = list(x.shape)
    shape[dh] += 2 * pad_h
    shape[dw] += 2 * pad_w
    r = x.new_full(shape, value)
    idx = [slice(None)] * 4
    idx[dh] = slice(pad_h, pad_h + x.shape[dh])
    idx[dw] = slice(pad_w, pad_w + x.shape[dw])
    r[tuple(idx)] = x
    return _emit(r, out)


def unpad(x: torch.Tensor, pad_h: int, pad_w: int, layout: str = "nhwc", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of :func:`pad`."""
    dh, dw = _hw_dims(x, layout)
    if x.shape[dh] <= 2 * pad_h or x.shape[dw] <= 2 * pad_w:
        raise ValueError("padding larger than the tensor")
    return crop(x, pad_h, pad_w, x.shape[dh] - pad_h - 1, x.shape[dw] - pad_w - 1, layout, out)


def crop(x: torch.Tensor, start_h: int, start_w: int, end_h: int, end_w: int, layout: str = "nhwc",
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``start_h..end_h`` and columns ``start_w..end_w``, both ends INCLUSIVE (the reference's convention,
    tensor_ops.hpp:313-363)."""
    dh, dw = _hw_dims(x, layout)
    if not (0 <= start_h <= end_h < x.shape[dh] and 0 <= start_w <= end_w < x.shape[dw]):
        raise ValueError("crop window outside the tensor")
    idx = [slice(None)] * 4
    idx[dh] = slice(start_h, end_h + 1)
    idx[dw] = slice(start_w, end_w + 1)
    return _emit(x[tuple(idx)], out)


# ------------------------------------------------------------------------------- batch slicing
def slice_batch(x: torch.Tensor, start: int, end: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Samples ``start`` (inclusive) to ``end`` (exclusive) of the leading dimension."""
    if not (0 <= start < end <= x.shape[0]):
        raise ValueError("batch range outside the tensor")
    return _emit(x[start:end], out)


def split(x: torch.Tensor, num_splits: int) -> List[torch.Tensor]:
    """``num_splits`` consecutive parts of the batch; the first ``batch % num_splits`` parts hold one sample more
    (micro-batching of the reference's coordinator, tensor_ops.hpp:418-474)."""
    n = x.shape[0]
    if num_splits <= 0 or num_splits > n:
        raise ValueError("invalid number of splits")
    base, extra = divmod(n, num_splits)
    parts, at = [], 0
    for i in range(num_splits):
        size = base + (1 if i < extra else 0)
        parts.append(x[at:at + size].contiguous())
        at += size
    return parts


# --------------------------------------------------------------------------------- transposes
def transpose_2d(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.dim() != 2:
        raise ValueError("expected a matrix")
    return _emit(x.t(), out)


def nchw_to_cnhw(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _emit(x.permute(1, 0, 2, 3), out)


def cnhw_to_nchw(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _emit(x.permute(1, 0, 2, 3), out)


def nchw_to_nhwc(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _emit(x.permute(0, 2, 3, 1), out)


def nhwc_to_nchw(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _emit(x.permute(0, 3, 1, 2), out)


# ------------------------------------------------------------------------ patch matrix and back
def im2col(x: torch.Tensor, kernel: Sequence[int], stride: Sequence[int] = (1, 1), pad_: Sequence[int] = (0, 0),
           layout: str = "nhwc") -> torch.Tensor:
    """Patch matrix ``[N * OH * OW, KH * KW * C]`` (taps outermost, channels innermost: the K order of the KRSC
    filters). bf16 NHWC tensors on a GPU use this package's kernel, everything else a gather in PyTorch."""
    kh, kw = kernel
    sh, sw = stride
    ph, pw = pad_
    if layout == "nchw":
        x = x.permute(0, 2, 3, 1)
    n, h, w, c = x.shape
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    if x.is_cuda and x.dtype == torch.bfloat16 and layout == "nhwc":
        from .conv import im2col as _k
        cols, kdim = _k(x.contiguous(), kh, kw, (sh, sw), (ph, pw), oh, ow)
        return cols[:, :kh * kw * c] if kdim != kh * kw * c else cols
    xp = torch.nn.functional.pad(x, (0, 0, pw, pw, ph, ph))
    taps = [xp[:, i:i + sh * (oh - 1) + 1:sh, j:j + sw * (ow - 1) + 1:sw, :] for i in range(kh) for j in range(kw)]
    return torch.stack(taps, 3).reshape(n * oh * ow, kh * kw * c).contiguous()


def col2im(cols: torch.Tensor, shape: Sequence[int], kernel: Sequence[int], stride: Sequence[int] = (1, 1),
           pad_: Sequence[int] = (0, 0), layout: str = "nhwc") -> torch.Tensor:
    """Adjoint of :func:`im2col`: every patch element is added back to the pixel it was taken from.
    ``shape`` is the image tensor's shape in ``layout``."""
    kh, kw = kernel
    sh, sw = stride
    ph, pw = pad_
    if layout == "nchw":
        n, c, h, w = shape
    else:
        n, h, w, c = shape
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    acc = torch.zeros(n, h + 2 * ph, w + 2 * pw, c, dtype=torch.float32, device=cols.device)
    v = cols.reshape(n, oh, ow, kh * kw, c).float()
    t = 0
    for i in range(kh):
        for j in range(kw):
            acc[:, i:i + sh * (oh - 1) + 1:sh, j:j + sw * (ow - 1) + 1:sw, :] += v[:, :, :, t, :]
            t += 1
    img = acc[:, ph:ph + h, pw:pw + w, :].to(cols.dtype)
    return (img.permute(0, 3, 1, 2) if layout == "nchw" else img).contiguous()


def check_equals(a: torch.Tensor, b: torch.Tensor, tolerance: float = 0.0) -> bool:
    return a.shape == b.shape and bool(((a.float() - b.float()).abs() <= tolerance).all())
