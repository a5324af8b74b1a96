"""Batch normalisation on CUDA (csrc/kernels/batchnorm.cu)."""
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
        vp, i, ll, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.tnnb_batchnorm_fwd.argtypes = [vp] * 9 + [ll, i, f, f, i, i, vp]
        lib.tnnb_batchnorm_bwd.argtypes = [vp] * 11 + [ll, i, i, vp]
        lib.tnnb_batchnorm_fwd.restype = lib.tnnb_batchnorm_bwd.restype = i
        lib.tnnb_batchnorm_fwd_res.argtypes = [vp] * 10 + [ll, i, f, f, i, i, vp]
        lib.tnnb_batchnorm_fwd_res.restype = i
        _DECL = True
    return lib


def _f32(t):
    if t.dtype != torch.float32:
        raise TypeError("batch-norm running statistics must be fp32 tensors (use the graph's master views)")
    return t


def _fwd(x, resid, *rest):
    """``tnnb_batchnorm_fwd`` or, with a residual operand, ``tnnb_batchnorm_fwd_res`` (y = relu?(bn(x) + resid))."""
    if resid is None:
        return _l().tnnb_batchnorm_fwd(_lib.ptr(x), *rest)
    if resid.shape != x.shape or resid.dtype != x.dtype:
        raise ValueError("the residual operand must have the shape and dtype of the batch-norm input")
    return _l().tnnb_batchnorm_fwd_res(_lib.ptr(x), _lib.ptr(resid.contiguous()), *rest)


def batchnorm_fwd_train(x, gamma, beta, run_mean, run_var, eps, momentum, relu, resid=None, post_add=False):
    C = x.shape[-1]
    M = x.numel() // C
    y = torch.empty_like(x)
    mean = torch.empty(C, dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    ws = torch.empty(2 * C, dtype=torch.float64, device=x.device)
    rc = _fwd(x, resid, _lib.ptr(y), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(ws), _lib.ptr(mean),
              _lib.ptr(rstd), _lib.ptr(_f32(run_mean)), _lib.ptr(_f32(run_var)), M, C, eps, momentum,
              int(relu) | (2 if (post_add and resid is not None) else 0), 1, _lib.stream())
    _lib.check_rc(rc, "batchnorm_fwd")
    LAUNCHES["count"] += 2
    return y, mean, rstd


def batchnorm_infer(x, gamma, beta, run_mean, run_var, eps, relu, resid=None, post_add=False):
    C = x.shape[-1]
    M = x.numel() // C
    y = torch.empty_like(x)
    rc = _fwd(x, resid, _lib.ptr(y), _lib.ptr(gamma), _lib.ptr(beta), None, None, None,
              _lib.ptr(_f32(run_mean)), _lib.ptr(_f32(run_var)), M, C, eps, 0.0,
              int(relu) | (2 if (post_add and resid is not None) else 0), 0, _lib.stream())
    _lib.check_rc(rc, "batchnorm_infer")
    LAUNCHES["count"] += 1
    return y


def batchnorm_bwd(dy, x, y, mean, rstd, gamma, dgamma, dbeta, relu, beta=None):
    """With a fused ReLU the kernels recompute the mask ``y > 0`` from ``x`` (same scale / shift arithmetic as the
    forward) when they know the layer's shift - ``beta`` given, or a non-affine layer - and then never read ``y``."""
    C = x.shape[-1]
    M = x.numel() // C
    dx = torch.empty_like(x)
    ws = torch.empty(2 * C, dtype=torch.float64, device=x.device)
    remask = relu and (beta is not None or gamma is None)
    rc = _l().tnnb_batchnorm_bwd(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(y if (relu and not remask) else None), _lib.ptr(gamma),
                                 _lib.ptr(beta if remask else None), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(ws), _lib.ptr(dx),
                                 _lib.ptr(dgamma), _lib.ptr(dbeta), M, C, int(relu), _lib.stream())
    _lib.check_rc(rc, "batchnorm_bwd")
    LAUNCHES["count"] += 2
    return dx
