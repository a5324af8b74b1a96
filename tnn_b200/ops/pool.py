"""Max / average pooling on CUDA (csrc/kernels/conv_pool.cu). The max-pool index is the
window-relative argmax stored as uint8 (the reference keeps an int32 tensor)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .gemm import LAUNCHES

_DECL = False


def _l():
    global _DECL
    lib = _lib.load()
    if not _DECL:
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.tnnb_pool_fwd.argtypes = [vp, vp, vp] + [i] * 11 + [vp]
        lib.tnnb_pool_bwd.argtypes = [vp, vp, vp] + [i] * 11 + [vp]
        lib.tnnb_pool_fwd.restype = lib.tnnb_pool_bwd.restype = i
        _DECL = True
    return lib


def pool2d_fwd(x, mode, pool, stride, pad, need_index=True):
    n, h, w, c = x.shape
    oh = (h + 2 * pad[0] - pool[0]) // stride[0] + 1
    ow = (w + 2 * pad[1] - pool[1]) // stride[1] + 1
    y = torch.empty(n, oh, ow, c, dtype=x.dtype, device=x.device)
    idx = torch.empty(n, oh, ow, c, dtype=torch.uint8, device=x.device) if (mode == "max" and need_index) else None
    rc = _l().tnnb_pool_fwd(_lib.ptr(x), _lib.ptr(y), _lib.ptr(idx), n, h, w, c, pool[0], pool[1], stride[0], stride[1], pad[0],
                            pad[1], 0 if mode == "max" else 1, _lib.stream())
    _lib.check_rc(rc, "pool_fwd")
    LAUNCHES["count"] += 1
    return y, idx


def pool2d_bwd(dy, idx, x_shape, mode, pool, stride, pad):
    n, h, w, c = x_shape
    dx = torch.empty(n, h, w, c, dtype=dy.dtype, device=dy.device)
    rc = _l().tnnb_pool_bwd(_lib.ptr(dy), _lib.ptr(idx), _lib.ptr(dx), n, h, w, c, pool[0], pool[1], stride[0], stride[1], pad[0],
                            pad[1], 0 if mode == "max" else 1, _lib.stream())
    _lib.check_rc(rc, "pool_bwd")
    LAUNCHES["count"] += 1
    return dx
