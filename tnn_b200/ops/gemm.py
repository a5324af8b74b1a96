"""bf16 GEMM with fused epilogues (tcgen05 kernel on CUDA, torch math on CPU).

``gemm(a, b)`` computes ``op(a) @ op(b).T`` where each operand is either
``[rows, K]`` (K-major, the default) or ``[K, rows]`` (``a_t`` / ``b_t``).
That covers the forward, dgrad and wgrad products of a dense layer
(reference: src/nn/engines/cuda_engine.cu:1652-1707) without a transpose pass.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

EPI_BIAS, EPI_GELU, EPI_DGELU, EPI_RESID, EPI_RELU, EPI_ATOMIC, EPI_OUT_F32, EPI_ACCUM = 1, 2, 4, 8, 16, 32, 64, 128

LAUNCHES = {"count": 0}


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def gelu_tanh_grad(x: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def _ld(t: torch.Tensor) -> int:
    assert t.dim() == 2 and t.stride(1) == 1, "operands must be 2-D with a unit inner stride"
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """An operand the TMA descriptors accept: unit inner stride, row pitch and base address multiples of 16 bytes.
    Tensors produced by the layers already are (their buffers are allocated with padded pitches); anything else -
    a gradient handed in by user code, an odd-width slice - is copied once into a padded buffer."""
    per16 = 16 // t.element_size()
    if t.dim() == 2 and t.stride(1) == 1 and t.data_ptr() % 16 == 0 and _ld(t) % per16 == 0:
        return t
    pitch = (t.shape[1] + per16 - 1) // per16 * per16
    buf = torch.zeros((t.shape[0], pitch), dtype=t.dtype, device=t.device)
    buf[:, :t.shape[1]].copy_(t)
    return buf[:, :t.shape[1]]


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         bias: Optional[torch.Tensor] = None, gelu: bool = False, save_preact: Optional[torch.Tensor] = None,
         dgelu_of: Optional[torch.Tensor] = None, relu: bool = False, residual: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         atomic: bool = False, split_k: int = 0, force_bn: int = 0) -> torch.Tensor:
    """``out = epilogue(op(a) @ op(b).T)``.

    a: ``[M,K]`` (or ``[K,M]`` with ``a_t``); b: ``[N,K]`` (or ``[K,N]`` with ``b_t``).
    ``atomic`` adds into an fp32 ``out`` with red.add and enables split-K (used by wgrad,
    whose reduction dimension is the batch).
    """
    M = a.shape[1] if a_t else a.shape[0]
    K = a.shape[0] if a_t else a.shape[1]
    N = b.shape[1] if b_t else b.shape[0]
    Kb = b.shape[0] if b_t else b.shape[1]
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if atomic:
        assert out is not None and out.dtype == torch.float32
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    assert out.shape == (M, N)

    if not a.is_cuda:
        A = (a.t() if a_t else a).float()
        B = (b.t() if b_t else b).float()
        r = A @ B.t()
        if bias is not None:
            r = r + bias.float()
        if gelu:
            if save_preact is not None:
                save_preact.copy_(r.to(save_preact.dtype))
                r = save_preact.float()
            r = gelu_tanh(r)
        if dgelu_of is not None:
            r = r * gelu_tanh_grad(dgelu_of.float())
        if relu:
            r = torch.relu(r)
        if residual is not None:
            r = r + residual.float()
        if atomic or accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    a, b = _tma_ready(a), _tma_ready(b)
    flags = 0
    if bias is not None:
        flags |= EPI_BIAS
        assert bias.dtype == torch.bfloat16 and bias.numel() == N
    if gelu:
        flags |= EPI_GELU
    if dgelu_of is not None:
        flags |= EPI_DGELU
    if relu:
        flags |= EPI_RELU
    if residual is not None:
        flags |= EPI_RESID
        assert residual.dtype == torch.bfloat16
    if atomic:
        flags |= EPI_ATOMIC
    elif out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    if accumulate and not atomic:
        flags |= EPI_ACCUM
    aux = save_preact if gelu else dgelu_of
    lib = _lib.load()
    rc = lib.tnnb_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, int(a_t), int(b_t), _ld(a), _ld(b), _ld(out),
        _lib.ptr(bias), _lib.ptr(dgelu_of), _lib.ptr(save_preact if gelu else None),
        _ld(aux) if aux is not None else 0, _lib.ptr(residual), _ld(residual) if residual is not None else 0,
        flags, split_k, force_bn, _lib.ptr(_lib.status_word(a.device)), _lib.stream())
    _lib.check_rc(rc, "tnnb_gemm_bf16")
    LAUNCHES["count"] += 1
    return out


_BATCHED_DECLARED = False


def gemm_batched(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
                 out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i] = op(a[i]) @ op(b[i]).T`` for every ``i`` of the leading dimension, in one launch of the batched
    tcgen05 kernel. a: ``[G, M, K]`` (``[G, K, M]`` with ``a_t``), b: ``[G, N, K]`` (``[G, K, N]`` with ``b_t``); the
    last dimension must be contiguous, the row pitch a multiple of 8 elements. ``out``: ``[G, M, N]`` bf16 or fp32,
    possibly a view with a padded row pitch."""
    G = a.shape[0]
    M = a.shape[2] if a_t else a.shape[1]
    K = a.shape[1] if a_t else a.shape[2]
    N = b.shape[2] if b_t else b.shape[1]
    assert b.shape[0] == G and (b.shape[1] if b_t else b.shape[2]) == K
    if out is None:
        out = torch.empty(G, M, N, dtype=out_dtype or a.dtype, device=a.device)
    if not a.is_cuda:
        A = (a.transpose(1, 2) if a_t else a).float()
        B = (b.transpose(1, 2) if b_t else b).float()
        out.copy_((A @ B.transpose(1, 2)).to(out.dtype))
        return out
    global _BATCHED_DECLARED
    lib = _lib.load()
    if not _BATCHED_DECLARED:
        import ctypes
        vp, ll, i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
        lib.tnnb_gemm_bf16_batched.argtypes = [vp, vp, vp, i, i, i, i, i, ll, ll, ll, i, ll, ll, ll, i, vp, vp]
        lib.tnnb_gemm_bf16_batched.restype = i
        _BATCHED_DECLARED = True
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(2) == 1 and b.stride(2) == 1 and out.stride(2) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    rc = lib.tnnb_gemm_bf16_batched(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, int(a_t), int(b_t), a.stride(1), b.stride(1),
                                    out.stride(1), G, a.stride(0), b.stride(0), out.stride(0),
                                    64 if out.dtype == torch.float32 else 0, _lib.ptr(_lib.status_word(a.device)), _lib.stream())
    _lib.check_rc(rc, "tnnb_gemm_bf16_batched")
    LAUNCHES["count"] += 1
    return out
