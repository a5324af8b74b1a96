"""Raw (non-autograd) operator entry points.

Each function runs the sm_100a kernel when its tensors are on a CUDA device and an
equivalent fp32 torch computation otherwise (the CPU path doubles as the numerical
reference in the tests). Nothing here falls back to torch for CUDA tensors.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .gemm import LAUNCHES, gelu_tanh, gelu_tanh_grad

ACT_KINDS = {"relu": 0, "gelu": 1, "elu": 2, "leaky_relu": 3, "sigmoid": 4, "tanh": 5, "linear": 6}
_M64 = (1 << 64) - 1


def _count(n=1):
    LAUNCHES["count"] += n


# ----------------------------------------------------------------------------- RNG
def hash_uniform(seed: int, idx: torch.Tensor) -> torch.Tensor:
    """Counter-based uniform in [0,1) identical to the device function of the same name."""
    def lsr(x, k):
        return (x >> k) & ((1 << (64 - k)) - 1)

    def c(v):  # python int -> wrapped int64 constant
        v &= _M64
        return v - (1 << 64) if v >= (1 << 63) else v

    z = idx.to(torch.int64) * c(0x9E3779B97F4A7C15) + c(seed)
    z = (z ^ lsr(z, 30)) * c(0xBF58476D1CE4E5B9)
    z = (z ^ lsr(z, 27)) * c(0x94D049BB133111EB)
    z = z ^ lsr(z, 31)
    return lsr(z, 40).to(torch.float32) * (1.0 / 16777216.0)


# Optional device-resident step counter added to every dropout seed (see mix_seed in
# csrc/kernels/ptx.cuh): set ``SEED_OFF["tensor"]`` to a 1-element int64 tensor that is
# bumped once per training step so that a captured CUDA graph draws fresh masks per replay.
SEED_OFF = {"tensor": None}


def _seed_off_ptr():
    return _lib.ptr(SEED_OFF["tensor"])


def _eff_seed(seed: int) -> int:
    t = SEED_OFF["tensor"]
    if t is None:
        return seed
    return (seed + int(t.item()) * 0xD1B54A32D192ED03) & _M64


def dropout_mask(shape, p: float, seed: int, device="cpu") -> torch.Tensor:
    """Keep mask of a flat tensor, identical to the device function ``dropout_keep8`` (csrc/kernels/ptx.cuh): the
    eight elements of chunk ``i // 8`` take the eight 16-bit fields of two 64-bit words mixed from (seed, chunk) and
    are kept when their field is ``>= round(p * 65536)``."""
    import numpy as np

    def lsr(x, k):
        return (x >> k) & ((1 << (64 - k)) - 1)

    def c(v):
        v &= _M64
        return v - (1 << 64) if v >= (1 << 63) else v

    n = int(math.prod(shape))
    thr = int(np.float32(p) * np.float32(65536.0) + np.float32(0.5))
    chunk = torch.arange((n + 7) // 8, device=device, dtype=torch.int64)
    z = chunk * c(0x9E3779B97F4A7C15) + c(seed)
    z = (z ^ lsr(z, 30)) * c(0xBF58476D1CE4E5B9)
    z = (z ^ lsr(z, 27)) * c(0x94D049BB133111EB)
    z = z ^ lsr(z, 31)
    w = (z ^ lsr(z, 29)) * c(0xD6E8FEB86659FD93)
    w = w ^ lsr(w, 32)
    fields = [lsr(z, 16 * k) & 0xFFFF for k in range(4)] + [lsr(w, 16 * k) & 0xFFFF for k in range(4)]
    keep = torch.stack(fields, dim=1) >= thr          # [chunks, 8]
    return keep.reshape(-1)[:n].reshape(shape)


# ---------------------------------------------------------------------- element-wise
def act_fwd(x: torch.Tensor, kind: str, alpha: float = 0.0) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x.contiguous()
        y = torch.empty_like(x)
        rc = _lib.load().tnnb_act_fwd(_lib.ptr(x), _lib.ptr(y), x.numel(), ACT_KINDS[kind], alpha, _lib.stream())
        _lib.check_rc(rc, "act_fwd")
        _count()
        return y
    xf = x.float()
    if kind == "relu":
        r = torch.relu(xf)
    elif kind == "gelu":
        r = gelu_tanh(xf)
    elif kind == "elu":
        r = torch.where(xf > 0, xf, alpha * (torch.exp(xf) - 1))
    elif kind == "leaky_relu":
        r = torch.where(xf > 0, xf, alpha * xf)
    elif kind == "sigmoid":
        r = torch.sigmoid(xf)
    elif kind == "tanh":
        r = torch.tanh(xf)
    else:
        r = xf
    return r.to(x.dtype)


def act_bwd(x: torch.Tensor, dy: torch.Tensor, kind: str, alpha: float = 0.0) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        x, dy = x.contiguous(), dy.contiguous()
        dx = torch.empty_like(x)
        rc = _lib.load().tnnb_act_bwd(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dx), x.numel(), ACT_KINDS[kind], alpha,
                                      _lib.stream())
        _lib.check_rc(rc, "act_bwd")
        _count()
        return dx
    xf = x.float()
    if kind == "relu":
        g = (xf > 0).float()
    elif kind == "gelu":
        g = gelu_tanh_grad(xf)
    elif kind == "elu":
        g = torch.where(xf > 0, torch.ones_like(xf), alpha * torch.exp(xf))
    elif kind == "leaky_relu":
        g = torch.where(xf > 0, torch.ones_like(xf), torch.full_like(xf, alpha))
    elif kind == "sigmoid":
        s = torch.sigmoid(xf)
        g = s * (1 - s)
    elif kind == "tanh":
        g = 1 - torch.tanh(xf) ** 2
    else:
        g = torch.ones_like(xf)
    return (dy.float() * g).to(x.dtype)


_BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3}


def binary(a: torch.Tensor, b: torch.Tensor, op: str, relu: bool = False) -> torch.Tensor:
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape == b.shape:
        a, b = a.contiguous(), b.contiguous()
        o = torch.empty_like(a)
        rc = _lib.load().tnnb_binary(_lib.ptr(a), _lib.ptr(b), _lib.ptr(o), a.numel(), _BIN[op], int(relu),
                                     _lib.stream())
        _lib.check_rc(rc, "binary")
        _count()
        return o
    af, bf = a.float(), b.float()
    r = af + bf if op == "add" else af - bf if op == "sub" else af * bf if op == "mul" else af / bf
    if relu:
        r = torch.relu(r)
    return r.to(a.dtype)


def dropout(x: torch.Tensor, p: float, seed: int) -> torch.Tensor:
    """``keep ? x/(1-p) : 0`` with the mask regenerated from ``seed`` (apply to dy for the backward)."""
    if p <= 0.0:
        return x
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x.contiguous()
        y = torch.empty_like(x)
        rc = _lib.load().tnnb_dropout(_lib.ptr(x), _lib.ptr(y), x.numel(), p, seed & _M64, _seed_off_ptr(), _lib.stream())
        _lib.check_rc(rc, "dropout")
        _count()
        return y
    m = dropout_mask(x.shape, p, _eff_seed(seed),x.device)
    return torch.where(m, x.float() / (1 - p), torch.zeros((), device=x.device)).to(x.dtype)


def embedding_fwd(ids: torch.Tensor, wte: torch.Tensor, wpe: Optional[torch.Tensor], seq_len: int,
                  padding_idx: int, p: float, seed: int) -> torch.Tensor:
    """``out[r] = dropout(wte[ids[r]] + wpe[r % seq_len])`` for flattened ids (int64)."""
    rows, E = ids.numel(), wte.shape[1]
    ids = ids.reshape(-1).to(torch.int64).contiguous()
    if wte.is_cuda and wte.dtype == torch.bfloat16:
        out = torch.empty(rows, E, dtype=wte.dtype, device=wte.device)
        rc = _lib.load().tnnb_embedding_fwd(_lib.ptr(ids), _lib.ptr(wte), _lib.ptr(wpe), _lib.ptr(out), rows, E,
                                            seq_len, wte.shape[0], padding_idx, p, seed & _M64, _seed_off_ptr(), _lib.stream())
        _lib.check_rc(rc, "embedding_fwd")
        _count()
        return out
    safe = torch.where((ids < 0) | (ids >= wte.shape[0]), torch.zeros_like(ids), ids)
    o = wte.float()[safe]
    o = torch.where((ids == padding_idx)[:, None], torch.zeros_like(o), o)
    if wpe is not None:
        o = o + wpe.float()[torch.arange(rows, device=ids.device) % seq_len]
    if p > 0:
        o = torch.where(dropout_mask(o.shape, p, _eff_seed(seed),o.device), o / (1 - p), torch.zeros_like(o))
    return o.to(wte.dtype)


def embedding_bwd(ids: torch.Tensor, dy: torch.Tensor, dwte: Optional[torch.Tensor], dwpe: Optional[torch.Tensor],
                  seq_len: int, padding_idx: int, p: float, seed: int) -> None:
    """Scatter-add ``dropout'(dy)`` into fp32 ``dwte`` / ``dwpe``."""
    rows, E = dy.shape
    ids = ids.reshape(-1).to(torch.int64).contiguous()
    vocab = dwte.shape[0] if dwte is not None else 1 << 62
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        dy = dy.contiguous()
        rc = _lib.load().tnnb_embedding_bwd(_lib.ptr(ids), _lib.ptr(dy), _lib.ptr(dwte), _lib.ptr(dwpe), rows, E,
                                            seq_len, vocab, padding_idx, p, seed & _M64, _seed_off_ptr(), _lib.stream())
        _lib.check_rc(rc, "embedding_bwd")
        _count()
        return
    g = dy.float()
    if p > 0:
        g = torch.where(dropout_mask(g.shape, p, _eff_seed(seed),g.device), g / (1 - p), torch.zeros_like(g))
    if dwte is not None:
        safe = torch.where((ids < 0) | (ids >= vocab), torch.zeros_like(ids), ids)
        gg = torch.where((ids == padding_idx)[:, None], torch.zeros_like(g), g)
        dwte.index_add_(0, safe, gg.to(dwte.dtype))
    if dwpe is not None:
        dwpe.index_add_(0, torch.arange(rows, device=ids.device) % seq_len, g.to(dwpe.dtype))


def colsum_accum(dy: torch.Tensor, db: torch.Tensor) -> None:
    """``db (fp32) += dy.sum(0)`` - the bias gradient of a dense layer."""
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        assert db.dtype == torch.float32 and dy.stride(1) == 1
        rc = _lib.load().tnnb_colsum_accum(_lib.ptr(dy), dy.stride(0), _lib.ptr(db), dy.shape[0], dy.shape[1],
                                           _lib.stream())
        _lib.check_rc(rc, "colsum_accum")
        _count()
        return
    db.add_(dy.float().sum(0).to(db.dtype))


# ------------------------------------------------------------------------- layernorm
def _tp_tail(tp_pull, tp_push, device):
    """The trailing arguments of the tensor-parallel layer-norm entry points (csrc/kernels/layernorm.cu). ``tp_pull``
    is a reduce-scatter site whose inbox is added to the operand, ``tp_push`` a gather site whose peers receive the
    output (objects of tnn_b200.parallel.tp)."""
    pl = (tp_pull.n_pull, tp_pull.pull_src, _lib.ptr(tp_pull.arrived), _lib.ptr(tp_pull.pass_ctr), tp_pull.units) \
        if tp_pull is not None else (0, None, None, None, 0)
    ps = (tp_push.n_push, tp_push.push_dst, tp_push.push_ready, tp_push.push_row0, tp_push.ln_rows) if tp_push is not None \
        else (0, None, None, 0, 0)
    return (*pl, *ps, _lib.ptr(_lib.status_word(device)), _lib.stream())


_TP_DECLARED = False


def _declare_tp(lib):
    global _TP_DECLARED
    if _TP_DECLARED:
        return
    import ctypes
    vp, ll, i, u, f, ull = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_uint, ctypes.c_float, ctypes.c_ulonglong
    tail = [i, vp, vp, vp, u, i, vp, vp, ll, ll, vp, vp]
    lib.tnnb_layernorm_fwd_tp.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, i, f, f, ull, vp] + tail
    lib.tnnb_layernorm_fwd_tp.restype = i
    lib.tnnb_layernorm_bwd_tp.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ll, i, f, ull, vp] + tail
    lib.tnnb_layernorm_bwd_tp.restype = i
    lib.tnnb_layernorm_bwd_tp_db.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ll, i, f, ull, vp] + tail
    lib.tnnb_layernorm_bwd_tp_db.restype = i
    lib.tnnb_layernorm_bwd_db.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ll, i, f, ull, vp, vp]
    lib.tnnb_layernorm_bwd_db.restype = i
    _TP_DECLARED = True


def layernorm_fwd(x: torch.Tensor, delta: Optional[torch.Tensor], gamma: Optional[torch.Tensor],
                  beta: Optional[torch.Tensor], eps: float, p: float = 0.0, seed: int = 0,
                  h_out: Optional[torch.Tensor] = None, tp_pull=None, tp_push=None
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``x_out = x + dropout(delta)``; ``h = LN(x_out)``. Returns (x_out, h, mean, rstd); x is 2-D [rows, C].
    ``h_out`` (contiguous, same shape) receives ``h`` in place, e.g. rows of a symmetric gather buffer.
    Tensor parallelism (CUDA only): ``tp_pull`` adds the partial sums in a reduce-scatter site's inbox to ``delta``;
    ``tp_push`` also delivers ``h`` to the peers of a gather site (``h_out`` must then be that site's own rows)."""
    rows, C = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16:
        x = x.contiguous()
        h = h_out if h_out is not None else torch.empty_like(x)
        x_out = torch.empty_like(x) if delta is not None else None
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        if delta is not None:
            delta = delta.contiguous()
        lib = _lib.load()
        if tp_pull is not None or tp_push is not None:
            _declare_tp(lib)
            rc = lib.tnnb_layernorm_fwd_tp(_lib.ptr(x), _lib.ptr(delta), _lib.ptr(x_out), _lib.ptr(h), _lib.ptr(gamma),
                                           _lib.ptr(beta), _lib.ptr(mean), _lib.ptr(rstd), rows, C, eps, p, seed & _M64,
                                           _seed_off_ptr(), *_tp_tail(tp_pull, tp_push, x.device))
        else:
            rc = lib.tnnb_layernorm_fwd(_lib.ptr(x), _lib.ptr(delta), _lib.ptr(x_out), _lib.ptr(h),
                                        _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(mean), _lib.ptr(rstd), rows, C,
                                        eps, p, seed & _M64, _seed_off_ptr(), _lib.stream())
        _lib.check_rc(rc, "layernorm_fwd")
        _count()
        return (x_out if delta is not None else x), h, mean, rstd
    assert tp_pull is None and tp_push is None, "the tensor-parallel hand-offs exist on CUDA only"
    xf = x.float()
    if delta is not None:
        d = delta.float()
        if p > 0:
            d = torch.where(dropout_mask(d.shape, p, _eff_seed(seed),d.device), d / (1 - p), torch.zeros_like(d))
        xf = (xf + d).to(x.dtype).float()
    mean = xf.mean(1)
    var = xf.var(1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    hh = (xf - mean[:, None]) * rstd[:, None]
    if gamma is not None:
        hh = hh * gamma.float() + beta.float()
    return xf.to(x.dtype), hh.to(x.dtype), mean, rstd


def layernorm_bwd(dh: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor,
                  gamma: Optional[torch.Tensor], dres: Optional[torch.Tensor], want_ddelta: bool, p: float,
                  seed: int, dgamma: Optional[torch.Tensor], dbeta: Optional[torch.Tensor],
                  ddelta_out: Optional[torch.Tensor] = None, tp_pull=None, tp_push=None,
                  dbias: Optional[torch.Tensor] = None
                  ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (dx, ddelta); accumulates into fp32 dgamma/dbeta. ``ddelta_out`` receives ddelta in place.
    ``tp_pull`` / ``tp_push`` as in :func:`layernorm_fwd`: the pulled partial sums are added to ``dh``, ``ddelta`` is
    what gets pushed. ``dbias`` (fp32 [C]) += column sums of ddelta: the bias gradient of the dense layer whose output
    was added to the residual stream in front of this norm, computed in the same pass."""
    rows, C = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16:
        dh = dh.contiguous()
        dx = torch.empty_like(x)
        dd = (ddelta_out if ddelta_out is not None else torch.empty_like(x)) if want_ddelta else None
        if dres is not None:
            dres = dres.contiguous()
        lib = _lib.load()
        if dbias is not None and not want_ddelta:
            raise ValueError("dbias is the column sum of ddelta: want_ddelta must be set")
        if tp_pull is not None or tp_push is not None:
            _declare_tp(lib)
            if dbias is not None:
                rc = lib.tnnb_layernorm_bwd_tp_db(_lib.ptr(dh), _lib.ptr(x), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma),
                                                  _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dd), _lib.ptr(dgamma), _lib.ptr(dbeta),
                                                  _lib.ptr(dbias), rows, C, p, seed & _M64, _seed_off_ptr(),
                                                  *_tp_tail(tp_pull, tp_push, x.device))
            else:
                rc = lib.tnnb_layernorm_bwd_tp(_lib.ptr(dh), _lib.ptr(x), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma),
                                               _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dd), _lib.ptr(dgamma), _lib.ptr(dbeta),
                                               rows, C, p, seed & _M64, _seed_off_ptr(), *_tp_tail(tp_pull, tp_push, x.device))
        elif dbias is not None:
            _declare_tp(lib)
            rc = lib.tnnb_layernorm_bwd_db(_lib.ptr(dh), _lib.ptr(x), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma),
                                           _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dd), _lib.ptr(dgamma), _lib.ptr(dbeta),
                                           _lib.ptr(dbias), rows, C, p, seed & _M64, _seed_off_ptr(), _lib.stream())
        else:
            rc = lib.tnnb_layernorm_bwd(_lib.ptr(dh), _lib.ptr(x), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma),
                                        _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dd), _lib.ptr(dgamma),
                                        _lib.ptr(dbeta), rows, C, p, seed & _M64, _seed_off_ptr(), _lib.stream())
        _lib.check_rc(rc, "layernorm_bwd")
        _count()
        return dx, dd
    assert tp_pull is None and tp_push is None, "the tensor-parallel hand-offs exist on CUDA only"
    xh = (x.float() - mean[:, None]) * rstd[:, None]
    g = dh.float()
    if dgamma is not None:
        dgamma.add_((g * xh).sum(0).to(dgamma.dtype))
        dbeta.add_(g.sum(0).to(dbeta.dtype))
    dy = g * gamma.float() if gamma is not None else g
    s1 = dy.mean(1, keepdim=True)
    s2 = (dy * xh).mean(1, keepdim=True)
    dx = rstd[:, None] * (dy - s1 - xh * s2)
    if dres is not None:
        dx = dx + dres.float()
    dx = dx.to(x.dtype)
    dd = None
    if want_ddelta:
        dd = dx.float()
        if p > 0:
            dd = torch.where(dropout_mask(dd.shape, p, _eff_seed(seed),dd.device), dd / (1 - p), torch.zeros_like(dd))
        dd = dd.to(x.dtype)
        if dbias is not None:
            dbias.add_(dd.float().sum(0).to(dbias.dtype))
    return dx, dd


# ------------------------------------------------------------------------------ loss
def softmax_ce(logits: torch.Tensor, labels: torch.Tensor, vocab: int, grad_scale: Optional[float],
               loss_scale: float, grad_out: Optional[torch.Tensor] = None
               ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Fused log-softmax + NLL over rows of ``logits[:, :vocab]``.

    Returns (loss_sum (1,), corrects (1,) int32, grad or None). ``grad = (softmax-onehot)*grad_scale`` is
    written to ``grad_out`` (may be ``logits`` itself) when ``grad_scale`` is not None.
    """
    rows = logits.shape[0]
    labels = labels.reshape(-1).to(torch.int64)
    if logits.is_cuda and logits.dtype == torch.bfloat16:
        ld = logits.stride(0)
        if ld % 8 or ld < (vocab + 7) // 8 * 8 or logits.data_ptr() % 16:
            pad = (vocab + 7) // 8 * 8
            buf = torch.zeros(rows, pad, dtype=logits.dtype, device=logits.device)
            buf[:, :vocab] = logits[:, :vocab]
            logits = buf
            if grad_out is not None and (grad_out.stride(0) % 8 or grad_out.stride(0) < pad):
                grad_out = None
        grad = None
        if grad_scale is not None:
            if grad_out is not None:
                grad = grad_out
            else:
                grad = torch.empty(rows, logits.stride(0), dtype=logits.dtype, device=logits.device)
        loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
        corr = torch.zeros(1, dtype=torch.int32, device=logits.device)
        rc = _lib.load().tnnb_softmax_ce(_lib.ptr(logits), logits.stride(0), _lib.ptr(labels.contiguous()),
                                         _lib.ptr(grad), grad.stride(0) if grad is not None else 0, None,
                                         _lib.ptr(loss), _lib.ptr(corr), rows, vocab,
                                         grad_scale if grad_scale is not None else 0.0, loss_scale, _lib.stream())
        _lib.check_rc(rc, "softmax_ce")
        _count()
        return loss, corr, (grad[:, :vocab] if grad is not None else None)
    z = logits[:, :vocab].float()
    lse = torch.logsumexp(z, 1)
    loss = ((lse - z.gather(1, labels[:, None]).squeeze(1)).sum() * loss_scale).reshape(1)
    corr = (z.argmax(1) == labels).sum().to(torch.int32).reshape(1)
    grad = None
    if grad_scale is not None:
        g = torch.softmax(z, 1)
        g[torch.arange(rows), labels] -= 1
        grad = (g * grad_scale).to(logits.dtype)
        if grad_out is not None:
            grad_out[:, :vocab].copy_(grad)
            grad = grad_out[:, :vocab]
    return loss, corr, grad


# ------------------------------------------------------------------------- attention
# Head sizes other than 64 on a GPU: the fused flash kernels are specialised for D = 64 (every zoo model); other sizes
# (the reference's attention benchmark uses E 768 / 8 heads = 96, benchmarks/attention_benchmark.cpp:11-40) run as
# batched tcgen05 GEMMs over all heads of a group at once - scores, probabilities and the backward products - with the
# row softmax between them as a kernel of its own (csrc/kernels/elementwise.cu). The scores are materialised in fp32,
# so memory is O(S^2) per head; heads are processed in groups whose score buffers stay below about 1 GiB.
# D must be a multiple of 8 (16-byte rows for the TMA descriptors); S is free (rows are padded to a multiple of 8).
_ATTN_DECLARED = False


def _attn_lib():
    global _ATTN_DECLARED
    lib = _lib.load()
    if not _ATTN_DECLARED:
        import ctypes
        vp, ll, i, f = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
        lib.tnnb_attn_softmax_fwd.argtypes = [vp, vp, vp, ll, i, i, ll, f, i, vp]
        lib.tnnb_attn_softmax_fwd.restype = i
        lib.tnnb_attn_softmax_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ll, i, i, ll, f, i, vp]
        lib.tnnb_attn_softmax_bwd.restype = i
        _ATTN_DECLARED = True
    return lib


def _heads(x2d: torch.Tensor, B: int, S: int, H: int, D: int, part: int, parts: int) -> torch.Tensor:
    """``[B*S, parts*H*D]`` -> contiguous ``[B*H, S, D]`` of part ``part`` (q, k or v of a packed projection)."""
    return x2d.view(B, S, parts, H, D)[:, :, part].permute(0, 2, 1, 3).reshape(B * H, S, D).contiguous()


def _group(BH: int, S: int) -> int:
    per_head = max(1, S * ((S + 7) // 8 * 8) * 4)
    return max(1, min(BH, (1 << 30) // per_head))


def _attn_fwd_generic(qkv, B, S, H, D, causal, scale):
    from .gemm import gemm_batched
    if D % 8:
        raise ValueError(f"attention on a GPU needs a head size that is a multiple of 8 (got {D})")
    lib = _attn_lib()
    E, BH, Sp = H * D, B * H, (S + 7) // 8 * 8
    q, k, v = (_heads(qkv, B, S, H, D, i, 3) for i in range(3))
    o = torch.empty(BH, S, D, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(BH, S, dtype=torch.float32, device=qkv.device)
    G = _group(BH, S)
    sc = torch.empty(G, S, Sp, dtype=torch.float32, device=qkv.device)
    pr = torch.zeros(G, S, Sp, dtype=qkv.dtype, device=qkv.device)
    for g0 in range(0, BH, G):
        n = min(G, BH - g0)
        gemm_batched(q[g0:g0 + n], k[g0:g0 + n], out=sc[:n, :, :S])                         # scores
        rc = lib.tnnb_attn_softmax_fwd(_lib.ptr(sc), _lib.ptr(pr), _lib.ptr(lse[g0:g0 + n]), n * S, S, S, Sp, scale, int(causal),
                                       _lib.stream())
        _lib.check_rc(rc, "attn_softmax_fwd")
        _count()
        gemm_batched(pr[:n, :, :S], v[g0:g0 + n], b_t=True, out=o[g0:g0 + n])                # P V
    out = o.view(B, H, S, D).permute(0, 2, 1, 3).reshape(B * S, E).contiguous()
    return out, lse.view(B, H, S)


def _attn_bwd_generic(qkv, out, dout, lse, B, S, H, D, causal, scale):
    from .gemm import gemm_batched
    lib = _attn_lib()
    E, BH, Sp = H * D, B * H, (S + 7) // 8 * 8
    q, k, v = (_heads(qkv, B, S, H, D, i, 3) for i in range(3))
    do, o = _heads(dout, B, S, H, D, 0, 1), _heads(out, B, S, H, D, 0, 1)
    delta = (do.float() * o.float()).sum(-1)                                                 # [BH, S]
    lse2 = lse.reshape(BH, S).contiguous()
    dq, dk, dv = (torch.empty(BH, S, D, dtype=qkv.dtype, device=qkv.device) for _ in range(3))
    G = _group(BH, S)
    sc = torch.empty(G, S, Sp, dtype=torch.float32, device=qkv.device)
    dp = torch.empty(G, S, Sp, dtype=torch.float32, device=qkv.device)
    pr = torch.zeros(G, S, Sp, dtype=qkv.dtype, device=qkv.device)
    ds = torch.zeros(G, S, Sp, dtype=qkv.dtype, device=qkv.device)
    for g0 in range(0, BH, G):
        n = min(G, BH - g0)
        sl = slice(g0, g0 + n)
        gemm_batched(q[sl], k[sl], out=sc[:n, :, :S])                                        # scores again
        gemm_batched(do[sl], v[sl], out=dp[:n, :, :S])                                       # dP = dO V^T
        rc = lib.tnnb_attn_softmax_bwd(_lib.ptr(sc), _lib.ptr(dp), _lib.ptr(lse2[sl]), _lib.ptr(delta[sl]), _lib.ptr(pr),
                                       _lib.ptr(ds), n * S, S, S, Sp, scale, int(causal), _lib.stream())
        _lib.check_rc(rc, "attn_softmax_bwd")
        _count()
        gemm_batched(pr[:n, :, :S], do[sl], a_t=True, b_t=True, out=dv[sl])                  # dV = P^T dO
        gemm_batched(ds[:n, :, :S], k[sl], b_t=True, out=dq[sl])                             # dQ = dS K
        gemm_batched(ds[:n, :, :S], q[sl], a_t=True, b_t=True, out=dk[sl])                   # dK = dS^T Q
    pack = torch.stack([t.view(B, H, S, D).permute(0, 2, 1, 3).reshape(B * S, E) for t in (dq, dk, dv)], 1)
    return pack.reshape(B * S, 3 * E).contiguous()


def attn_fwd(qkv: torch.Tensor, B: int, S: int, H: int, D: int, causal: bool, scale: float
             ) -> Tuple[torch.Tensor, torch.Tensor]:
    """qkv: [B*S, 3*H*D] (q | k | v, heads contiguous). Returns (out [B*S, H*D], lse [B,H,S] in log2 units)."""
    E = H * D
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and D != 64:
        return _attn_fwd_generic(qkv.contiguous(), B, S, H, D, causal, scale)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16:
        qkv = qkv.contiguous()
        out = torch.empty(B * S, E, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B, H, S, dtype=torch.float32, device=qkv.device)
        rc = _lib.load().tnnb_attn_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), B, S, H, D, int(causal), scale,
                                       _lib.ptr(_lib.status_word(qkv.device)), _lib.stream())
        _lib.check_rc(rc, "attn_fwd")
        _count()
        return out, lse
    q, k, v = (t.reshape(B, S, H, D).permute(0, 2, 1, 3).float() for t in qkv.reshape(B * S, 3, E).unbind(1))
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=s.device), 1), float("-inf"))
    lse_n = torch.logsumexp(s, -1)
    pm = torch.exp(s - lse_n[..., None])
    o = (pm @ v).permute(0, 2, 1, 3).reshape(B * S, E)
    return o.to(qkv.dtype), lse_n * 1.4426950408889634


def attn_bwd(qkv: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor, B: int, S: int, H: int,
             D: int, causal: bool, scale: float) -> torch.Tensor:
    """Gradient with respect to the packed qkv, same layout as the input."""
    E = H * D
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and D != 64:
        return _attn_bwd_generic(qkv.contiguous(), out, dout.contiguous(), lse, B, S, H, D, causal, scale)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16:
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(B, H, S, dtype=torch.float32, device=qkv.device)
        dq_acc = torch.empty(B * S, E, dtype=torch.float32, device=qkv.device)  # zeroed by the entry point
        rc = _lib.load().tnnb_attn_bwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(delta),
                                       _lib.ptr(dq_acc), _lib.ptr(dqkv), B, S, H, D, int(causal), scale,
                                       _lib.ptr(_lib.status_word(qkv.device)), _lib.stream())
        _lib.check_rc(rc, "attn_bwd")
        _count(3)  # delta, fused dK/dV/dQ, dQ conversion (plus one memset node)
        return dqkv
    q, k, v = (t.reshape(B, S, H, D).permute(0, 2, 1, 3).float() for t in qkv.reshape(B * S, 3, E).unbind(1))
    do = dout.reshape(B, S, H, D).permute(0, 2, 1, 3).float()
    o = out.reshape(B, S, H, D).permute(0, 2, 1, 3).float()
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=s.device), 1), float("-inf"))
    pm = torch.exp2(s * 1.4426950408889634 - lse[..., None])
    dv = pm.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    ds = pm * (dp - (o * do).sum(-1, keepdim=True))
    dq = ds @ k * scale
    dk = ds.transpose(-1, -2) @ q * scale
    pack = torch.stack([t.permute(0, 2, 1, 3).reshape(B * S, E) for t in (dq, dk, dv)], 1)
    return pack.reshape(B * S, 3 * E).to(qkv.dtype)


# ------------------------------------------------------------------------ optimizers
def adam_step(master: torch.Tensor, p_lp: Optional[torch.Tensor], grad: torch.Tensor, m: torch.Tensor,
              v: torch.Tensor, lr: float, b1: float, b2: float, eps: float, wd: float, step: int,
              gscale: float = 1.0, hyper: Optional[torch.Tensor] = None) -> None:
    """Flat-buffer Adam (reference semantics: p -= lr*m^/(sqrt(v^)+eps) + wd*lr*p)."""
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    if master.is_cuda:
        rc = _lib.load().tnnb_adam_step(_lib.ptr(master), _lib.ptr(p_lp), _lib.ptr(grad), _lib.ptr(m), _lib.ptr(v),
                                        master.numel(), lr, b1, b2, eps, wd, bc1, bc2, gscale, _lib.ptr(hyper),
                                        _lib.stream())
        _lib.check_rc(rc, "adam_step")
        _count()
        return
    g = grad.float() * gscale
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    upd = lr * (m / bc1) / (torch.sqrt(v / bc2) + eps)
    master.sub_(upd + wd * lr * master)
    if p_lp is not None:
        p_lp.copy_(master.to(p_lp.dtype))


def sgd_step(master: torch.Tensor, p_lp: Optional[torch.Tensor], grad: torch.Tensor, vel: Optional[torch.Tensor],
             lr: float, momentum: float, gscale: float = 1.0, hyper: Optional[torch.Tensor] = None) -> None:
    """Flat-buffer SGD (reference semantics: v = mu*v - lr*g; p += v)."""
    if master.is_cuda:
        rc = _lib.load().tnnb_sgd_step(_lib.ptr(master), _lib.ptr(p_lp), _lib.ptr(grad), _lib.ptr(vel),
                                       master.numel(), lr, momentum, gscale, _lib.ptr(hyper), _lib.stream())
        _lib.check_rc(rc, "sgd_step")
        _count()
        return
    g = grad.float() * gscale
    if vel is not None:
        vel.mul_(momentum).sub_(g, alpha=lr)
        master.add_(vel)
    else:
        master.sub_(g, alpha=lr)
    if p_lp is not None:
        p_lp.copy_(master.to(p_lp.dtype))


# ------------------------------------------------------------------------------ conv
def _to_nchw(x):
    return x.permute(0, 3, 1, 2)


def conv2d_fwd(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], stride, pad,
               relu: bool = False, keep: Optional[dict] = None) -> torch.Tensor:
    """NHWC x [N,H,W,C] * OHWI w [O,KH,KW,C] -> [N,OH,OW,O] (zero padding, no dilation). On CUDA ``keep`` receives
    the patch matrix (``keep["cols"]``) for :func:`conv2d_wgrad`."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import conv
        return conv.conv2d_fwd(x, w, bias, stride, pad, relu, keep)
    y = torch.nn.functional.conv2d(_to_nchw(x).float(), w.permute(0, 3, 1, 2).float(),
                                   None if bias is None else bias.float(), stride, pad)
    if relu:
        y = torch.relu(y)
    return y.permute(0, 2, 3, 1).contiguous().to(x.dtype)


def conv2d_dgrad(dy: torch.Tensor, w: torch.Tensor, x_shape, stride, pad, add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Input gradient of a convolution; ``add`` is summed into it (fused into the GEMM epilogue for 1 x 1 filters)."""
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        from . import conv
        return conv.conv2d_dgrad(dy, w, x_shape, stride, pad, add)
    n, h, wd, c = x_shape
    dx = torch.nn.grad.conv2d_input((n, c, h, wd), w.permute(0, 3, 1, 2).float(), _to_nchw(dy).float(), stride, pad)
    dx = dx.permute(0, 2, 3, 1)
    if add is not None:
        dx = dx + add.float()
    return dx.contiguous().to(dy.dtype)


def conv2d_wgrad(x: torch.Tensor, dy: torch.Tensor, dw: torch.Tensor, stride, pad, cols: Optional[torch.Tensor] = None) -> None:
    """dw (fp32, [O,KH,KW,C]) += correlation of x with dy."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import conv
        return conv.conv2d_wgrad(x, dy, dw, stride, pad, cols)
    o, kh, kw, c = dw.shape
    g = torch.nn.grad.conv2d_weight(_to_nchw(x).float(), (o, c, kh, kw), _to_nchw(dy).float(), stride, pad)
    dw.add_(g.permute(0, 2, 3, 1).to(dw.dtype))


# ------------------------------------------------------------------------- batchnorm
def batchnorm_fwd_train(x, gamma, beta, run_mean, run_var, eps: float, momentum: float, relu: bool, resid=None,
                        post_add: bool = False):
    """Training-mode batch norm over all dims but the last; updates the running stats in place.
    Returns (y, mean, rstd) with fp32 statistics. With ``resid`` (shape of x) the result is ``relu?(bn(x) + resid)``:
    the closing add of a residual block done in the same pass; with ``post_add`` it is ``relu?(bn(x)) + resid`` (the
    add comes after the activation)."""
    C = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import norm
        return norm.batchnorm_fwd_train(x, gamma, beta, run_mean, run_var, eps, momentum, relu, resid, post_add)
    x2 = x.reshape(-1, C).float()
    M = x2.shape[0]
    mean = x2.mean(0)
    var = x2.var(0, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    y = (x2 - mean) * rstd
    if gamma is not None:
        y = y * gamma.float() + beta.float()
    if resid is not None and not post_add:
        y = y.to(x.dtype).float() + resid.reshape(-1, C).float()
    if relu:
        y = torch.relu(y)
    if resid is not None and post_add:
        y = y.to(x.dtype).float() + resid.reshape(-1, C).float()
    unb = var * (M / max(M - 1, 1))
    run_mean.copy_(((1 - momentum) * run_mean.float() + momentum * mean).to(run_mean.dtype))
    run_var.copy_(((1 - momentum) * run_var.float() + momentum * unb).to(run_var.dtype))
    return y.reshape(x.shape).to(x.dtype), mean, rstd


def batchnorm_infer(x, gamma, beta, run_mean, run_var, eps: float, relu: bool, resid=None, post_add: bool = False):
    C = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import norm
        return norm.batchnorm_infer(x, gamma, beta, run_mean, run_var, eps, relu, resid, post_add)
    scale = torch.rsqrt(run_var.float() + eps)
    shift = -run_mean.float() * scale
    if gamma is not None:
        scale = scale * gamma.float()
        shift = beta.float() - run_mean.float() * scale
    y = x.reshape(-1, C).float() * scale + shift
    if resid is not None and not post_add:
        y = y.to(x.dtype).float() + resid.reshape(-1, C).float()
    if relu:
        y = torch.relu(y)
    if resid is not None and post_add:
        y = y.to(x.dtype).float() + resid.reshape(-1, C).float()
    return y.reshape(x.shape).to(x.dtype)


def batchnorm_bwd(dy, x, y, mean, rstd, gamma, dgamma, dbeta, relu: bool, beta=None):
    """dx; dgamma/dbeta (fp32) accumulate. ``y`` is the saved post-ReLU output when relu is fused; the GPU kernels do
    not read it when ``beta`` is passed (they recompute the mask from ``x``)."""
    C = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import norm
        return norm.batchnorm_bwd(dy, x, y, mean, rstd, gamma, dgamma, dbeta, relu, beta)
    x2, g = x.reshape(-1, C).float(), dy.reshape(-1, C).float()
    M = x2.shape[0]
    if relu:
        g = g * (y.reshape(-1, C) > 0)
    xh = (x2 - mean) * rstd
    sg, sgx = g.sum(0), (g * xh).sum(0)
    if dgamma is not None:
        dgamma.add_(sgx.to(dgamma.dtype))
        dbeta.add_(sg.to(dbeta.dtype))
    gam = gamma.float() if gamma is not None else 1.0
    dx = gam * rstd / M * (M * g - sg - xh * sgx)
    return dx.reshape(x.shape).to(x.dtype)


# ------------------------------------------------------------------------------ pools
def _pool_windows(x, pool, stride, pad, fill):
    """[N,OH,OW,KH*KW,C] view of the windows plus a validity mask [1,OH,OW,KH*KW,1]."""
    n, h, w, c = x.shape
    xp = torch.nn.functional.pad(x.float(), (0, 0, pad[1], pad[1], pad[0], pad[0]), value=fill)
    valid = torch.nn.functional.pad(torch.ones(1, h, w, 1, device=x.device), (0, 0, pad[1], pad[1], pad[0], pad[0]))
    win = xp.unfold(1, pool[0], stride[0]).unfold(2, pool[1], stride[1])       # N,OH,OW,C,KH,KW
    vwin = valid.unfold(1, pool[0], stride[0]).unfold(2, pool[1], stride[1])
    oh, ow = win.shape[1], win.shape[2]
    win = win.permute(0, 1, 2, 4, 5, 3).reshape(n, oh, ow, pool[0] * pool[1], c)
    vwin = vwin.permute(0, 1, 2, 4, 5, 3).reshape(1, oh, ow, pool[0] * pool[1], 1)
    return win, vwin


def pool2d_fwd(x, mode: str, pool, stride, pad, need_index: bool = True):
    """Returns (y, idx). For max pooling idx is the window-relative argmax (int32, kh*pool_w+kw)."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from . import pool as pool_ops
        return pool_ops.pool2d_fwd(x, mode, pool, stride, pad, need_index)
    if mode == "max":
        win, vwin = _pool_windows(x, pool, stride, pad, float("-inf"))
        win = torch.where(vwin > 0, win, torch.full_like(win, float("-inf")))
        y, idx = win.max(3)
        return y.to(x.dtype), idx.to(torch.int32)
    win, vwin = _pool_windows(x, pool, stride, pad, 0.0)
    cnt = vwin.sum(3).clamp(min=1)
    return (win.sum(3) / cnt).to(x.dtype), None


def pool2d_bwd(dy, idx, x_shape, mode: str, pool, stride, pad):
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        from . import pool as pool_ops
        return pool_ops.pool2d_bwd(dy, idx, x_shape, mode, pool, stride, pad)
    n, h, w, c = x_shape
    oh, ow = dy.shape[1], dy.shape[2]
    dxp = torch.zeros(n, h + 2 * pad[0], w + 2 * pad[1], c)
    g = dy.float()
    if mode == "avg":
        _, vwin = _pool_windows(torch.zeros(1, h, w, 1), pool, stride, pad, 0.0)
        g = g / vwin.sum(3).clamp(min=1)
    for kh in range(pool[0]):
        for kw in range(pool[1]):
            sel = g if mode == "avg" else g * (idx == kh * pool[1] + kw)
            dxp[:, kh:kh + oh * stride[0]:stride[0], kw:kw + ow * stride[1]:stride[1], :] += sel
    return dxp[:, pad[0]:pad[0] + h, pad[1]:pad[1] + w, :].contiguous().to(dy.dtype)
