"""NHWC convolution on CUDA. Three routes, all ending on the tcgen05 tensor cores:

* 1x1, stride 1: a plain GEMM over the activations;
* channel counts that are multiples of 64: the implicit-GEMM kernels of ``csrc/kernels/conv_implicit.cu`` - TMA fetches
  shifted spatial boxes of the input straight into operand tiles, no patch matrix exists: forward, weight gradient,
  the data gradient of stride-1 layers (the forward kernel run on ``dy`` with the rotated filter) and the data
  gradient of strided layers (one launch of the forward kernel per parity class of input pixels, each a stride-1
  correlation of ``dy`` with the sub-filter of the taps that reach that class);
* 64 -> 64 channels, stride 1, filters up to 3 x 3 (ResNet-50's first stage): forward / data gradient and weight
  gradient kernels that load ONE input window with its halo per 16 x 8 pixel tile and address every filter tap
  inside it by moving the operand descriptor;
* everything else (the 3-channel stem, channel counts that are not multiples of 64): im2col / col2im kernels around
  the GEMM.

Reference semantics: src/nn/engines/cpu_engine.cpp:617-734; the reference itself calls cuDNN conv graphs."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib
from .gemm import LAUNCHES, gemm

_DECL = False


def _lib_conv():
    global _DECL
    lib = _lib.load()
    if not _DECL:
        vp, i = ctypes.c_void_p, ctypes.c_int
        for name in ("tnnb_im2col", "tnnb_col2im"):
            getattr(lib, name).argtypes = [vp, vp] + [i] * 11 + [vp]
            getattr(lib, name).restype = i
        lib.tnnb_conv2d_fwd_implicit.argtypes = [vp, vp, vp, vp] + [i] * 12 + [vp, vp]
        lib.tnnb_conv2d_fwd_implicit.restype = i
        lib.tnnb_conv2d_fwd_implicit_strided.argtypes = [vp, vp, vp] + [i] * 17 + [vp, vp]
        lib.tnnb_conv2d_fwd_implicit_strided.restype = i
        lib.tnnb_conv2d_fwd_halo.argtypes = [vp, vp, vp, vp] + [i] * 10 + [vp, vp]
        lib.tnnb_conv2d_fwd_halo.restype = i
        lib.tnnb_conv2d_wgrad_halo.argtypes = [vp, vp, vp] + [i] * 9 + [vp, vp]
        lib.tnnb_conv2d_wgrad_halo.restype = i
        lib.tnnb_conv2d_wgrad_implicit.argtypes = [vp, vp, vp] + [i] * 11 + [vp, vp]
        lib.tnnb_conv2d_wgrad_implicit.restype = i
        _DECL = True
    return lib


def _implicit_ok(c_in: int, c_out: int) -> bool:
    return c_in % 64 == 0 and c_out % 64 == 0


def _fwd_implicit(x, w, bias, stride, pad, relu):
    n, h, wd, c = x.shape
    o, kh, kw, _ = w.shape
    oh = (h + 2 * pad[0] - kh) // stride[0] + 1
    ow = (wd + 2 * pad[1] - kw) // stride[1] + 1
    y = torch.empty(n, oh, ow, o, dtype=x.dtype, device=x.device)
    if (c == 64 and o == 64 and tuple(stride) == (1, 1) and kh <= 3 and kw <= 3 and kh * kw > 1 and pad[0] >= 0 and pad[1] >= 0
            and os.environ.get("TNNB_CONV_HALO", "1") != "0"):
        # 64-channel layers: the input tile is loaded once with its halo instead of once per filter tap
        rc = _lib_conv().tnnb_conv2d_fwd_halo(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(y), n, h, wd, c, o, kh, kw, pad[0],
                                              pad[1], int(relu), _lib.ptr(_lib.status_word(x.device)), _lib.stream())
        _lib.check_rc(rc, "conv2d_fwd_halo")
        LAUNCHES["count"] += 1
        return y
    rc = _lib_conv().tnnb_conv2d_fwd_implicit(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(y), n, h, wd, c, o, kh, kw, stride[0],
                                              stride[1], pad[0], pad[1], int(relu), _lib.ptr(_lib.status_word(x.device)), _lib.stream())
    _lib.check_rc(rc, "conv2d_fwd_implicit")
    LAUNCHES["count"] += 1
    return y


def _geom(x_shape, w_shape, stride, pad):
    n, h, w, c = x_shape
    o, kh, kw, _ = w_shape
    oh = (h + 2 * pad[0] - kh) // stride[0] + 1
    ow = (w + 2 * pad[1] - kw) // stride[1] + 1
    return n, h, w, c, o, kh, kw, oh, ow


def _is_pointwise(kh, kw, stride, pad):
    return kh == 1 and kw == 1 and stride == (1, 1) and pad == (0, 0)


def im2col(x: torch.Tensor, kh, kw, stride, pad, oh, ow) -> Tuple[torch.Tensor, int]:
    n, h, w, c = x.shape
    K = kh * kw * c
    kld = (K + 7) // 8 * 8
    cols = torch.empty(n * oh * ow, kld, dtype=x.dtype, device=x.device)
    rc = _lib_conv().tnnb_im2col(_lib.ptr(x), _lib.ptr(cols), n, h, w, c, kh, kw, stride[0], stride[1], pad[0], pad[1], kld,
                                 _lib.stream())
    _lib.check_rc(rc, "im2col")
    LAUNCHES["count"] += 1
    return cols, K


def _w2d(w: torch.Tensor, K: int) -> torch.Tensor:
    """[O, KH*KW*C] view of the weights; padded to a multiple of 8 columns when TMA needs it."""
    w2 = w.reshape(w.shape[0], K)
    if K % 8 == 0:
        return w2
    pad = torch.zeros(w.shape[0], (K + 7) // 8 * 8, dtype=w.dtype, device=w.device)
    pad[:, :K] = w2
    return pad[:, :K]


def conv2d_fwd(x, w, bias, stride, pad, relu=False, keep=None):
    """``keep`` (a dict) receives the patch matrix under ``"cols"`` so that the weight-gradient pass can reuse
    it instead of gathering the patches a second time (it costs memory, not bandwidth)."""
    stride, pad = tuple(stride), tuple(pad)
    n, h, wd, c, o, kh, kw, oh, ow = _geom(x.shape, w.shape, stride, pad)
    if _is_pointwise(kh, kw, stride, pad) and c % 8 == 0:
        a, K = x.reshape(-1, c), c
    elif _implicit_ok(c, o) and x.is_contiguous() and w.is_contiguous():
        return _fwd_implicit(x, w, bias, stride, pad, relu)
    else:
        cols, K = im2col(x, kh, kw, stride, pad, oh, ow)
        a = cols[:, :K]
        if keep is not None:
            keep["cols"] = cols
    y = gemm(a, _w2d(w, K), bias=bias, relu=relu)
    return y.view(n, oh, ow, o)


def conv2d_dgrad(dy, w, x_shape, stride, pad, add=None):
    """Gradient with respect to the input. ``add`` (same shape as the result): another contribution to the same
    gradient - the shortcut branch of a residual block - which the 1 x 1 case adds in the GEMM epilogue instead of
    leaving it to a separate three-tensor pass."""
    stride, pad = tuple(stride), tuple(pad)
    n, h, wd, c, o, kh, kw, oh, ow = _geom(x_shape, w.shape, stride, pad)
    dy2 = dy.reshape(-1, o)
    K = kh * kw * c
    if _is_pointwise(kh, kw, stride, pad) and c % 8 == 0:
        res = add.reshape(-1, c) if add is not None and add.is_contiguous() else None
        dx = gemm(dy2, w.reshape(o, K), b_t=True, residual=res).view(n, h, wd, c)
        if add is not None and res is None:
            dx = raw_binary_add(dx, add)
        return dx
    if add is not None:
        return raw_binary_add(conv2d_dgrad(dy, w, x_shape, stride, pad), add)
    if stride == (1, 1) and _implicit_ok(o, c) and dy.is_contiguous() and kh - 1 - pad[0] >= 0 and kw - 1 - pad[1] >= 0:
        # dx = conv(dy, filter rotated by 180 degrees with its channel axes swapped), padding k - 1 - p
        w_rot = w.flip(1, 2).permute(3, 1, 2, 0).contiguous()
        return _fwd_implicit(dy, w_rot, None, (1, 1), (kh - 1 - pad[0], kw - 1 - pad[1]), False)
    if (stride[0] > 1 or stride[1] > 1) and _implicit_ok(o, c) and dy.is_contiguous():
        return _dgrad_strided_implicit(dy, w, x_shape, stride, pad)
    kld = (K + 7) // 8 * 8
    dcols = torch.empty(dy2.shape[0], kld, dtype=dy.dtype, device=dy.device)
    gemm(dy2, _w2d(w, K), b_t=True, out=dcols[:, :K])
    dx = torch.empty(n, h, wd, c, dtype=dy.dtype, device=dy.device)
    rc = _lib_conv().tnnb_col2im(_lib.ptr(dcols), _lib.ptr(dx), n, h, wd, c, kh, kw, stride[0], stride[1], pad[0], pad[1], kld,
                                 _lib.stream())
    _lib.check_rc(rc, "col2im")
    LAUNCHES["count"] += 1
    return dx


def _parity_classes(size: int, k: int, s: int, p: int):
    """Input positions ``s * i + a`` (a = 0 .. s-1) of a strided convolution receive gradient only through the filter
    taps ``kh = r + s * m`` with ``r = (a + p) % s``, from output position ``i + q - m`` (``q = (a + p - r) / s``).
    Per class: (a, number of positions, taps in the order of ascending output position, padding of the equivalent
    stride-1 correlation over the output gradient)."""
    out = []
    for a in range(s):
        r = (a + p) % s
        nt = 0 if r >= k else (k - r + s - 1) // s
        q = (a + p - r) // s
        taps = [r + s * (nt - 1 - u) for u in range(nt)]  # = reversed(range(r, k, s))
        out.append((a, (size - a + s - 1) // s, taps, (nt - 1) - q))
    return out


def _dgrad_strided_implicit(dy, w, x_shape, stride, pad):
    """Data gradient of a strided convolution without a patch matrix: the input pixels fall into
    ``stride_h * stride_w`` parity classes, and each class is a stride-1 correlation of ``dy`` with the sub-filter of
    the taps that reach it - one launch of the implicit-GEMM forward kernel per class, writing every
    ``stride``-th pixel of ``dx``. Classes no tap reaches (1 x 1 filters) stay zero."""
    n, h, wd, c = x_shape
    o, kh, kw, _ = w.shape
    oh, ow = dy.shape[1], dy.shape[2]
    ch, cw = _parity_classes(h, kh, stride[0], pad[0]), _parity_classes(wd, kw, stride[1], pad[1])
    full = all(t for _, _, t, _ in ch) and all(t for _, _, t, _ in cw)
    dx = (torch.empty if full else torch.zeros)(n, h, wd, c, dtype=dy.dtype, device=dy.device)
    lib = _lib_conv()
    for a, hc, khs, phc in ch:
        for b, wc, kws, pwc in cw:
            if not khs or not kws or hc <= 0 or wc <= 0:
                continue
            # filter of the equivalent correlation: [C, taps_h, taps_w, O]
            # taps descend by the stride: a strided slice, flipped (no index tensors: this runs inside captured steps)
            w_sub = w[:, khs[-1]::stride[0], kws[-1]::stride[1]].flip(1, 2).permute(3, 1, 2, 0).contiguous()
            rc = lib.tnnb_conv2d_fwd_implicit_strided(_lib.ptr(dy), _lib.ptr(w_sub), _lib.ptr(dx), n, oh, ow, o, c, len(khs),
                                                      len(kws), phc, pwc, hc, wc, h, wd, stride[0], stride[1], a, b,
                                                      _lib.ptr(_lib.status_word(dy.device)), _lib.stream())
            _lib.check_rc(rc, "conv2d_fwd_implicit_strided")
            LAUNCHES["count"] += 1
    return dx


def raw_binary_add(a, b):
    from . import raw
    return raw.binary(a.contiguous(), b.contiguous(), "add")


def conv2d_wgrad(x, dy, dw, stride, pad, cols=None):
    stride, pad = tuple(stride), tuple(pad)
    n, h, wd, c, o, kh, kw, oh, ow = _geom(x.shape, dw.shape, stride, pad)
    dy2 = dy.reshape(-1, o)
    K = kh * kw * c
    if _is_pointwise(kh, kw, stride, pad) and c % 8 == 0:
        a = x.reshape(-1, c)
    elif cols is None and _implicit_ok(c, o) and dw.dtype == torch.float32 and dw.is_contiguous() and x.is_contiguous() \
            and dy.is_contiguous():
        if (c == 64 and o == 64 and stride == (1, 1) and kh <= 3 and kw <= 3 and kh * kw > 1 and pad[0] >= 0 and pad[1] >= 0
                and os.environ.get("TNNB_CONV_HALO", "1") != "0"):
            # 64-channel layers: one input window per pixel tile serves every filter tap
            rc = _lib_conv().tnnb_conv2d_wgrad_halo(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), n, h, wd, c, o, kh, kw, pad[0], pad[1],
                                                    _lib.ptr(_lib.status_word(x.device)), _lib.stream())
            _lib.check_rc(rc, "conv2d_wgrad_halo")
            LAUNCHES["count"] += 1
            return
        rc = _lib_conv().tnnb_conv2d_wgrad_implicit(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), n, h, wd, c, o, kh, kw, stride[0], stride[1],
                                                    pad[0], pad[1], _lib.ptr(_lib.status_word(x.device)), _lib.stream())
        _lib.check_rc(rc, "conv2d_wgrad_implicit")
        LAUNCHES["count"] += 1
        return
    else:
        if cols is None:
            cols, _ = im2col(x, kh, kw, stride, pad, oh, ow)
        a = cols[:, :K]
    if K % 4 == 0:
        gemm(dy2, a, a_t=True, b_t=True, out=dw.view(o, K), atomic=True)
    else:
        tmp = torch.zeros(o, (K + 7) // 8 * 8, dtype=torch.float32, device=dw.device)
        gemm(dy2, a, a_t=True, b_t=True, out=tmp[:, :K], atomic=True)
        dw.view(o, K).add_(tmp[:, :K])
