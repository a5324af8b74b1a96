"""The element-wise / reduction API of the reference's ``ops`` namespace (include/ops/ops.hpp:19-864), by name.

bf16 CUDA tensors go through this package's kernels where one exists (the binary operations); everything else is a
single PyTorch call on whatever device the tensors live on. All functions return their result; ``out=`` variants
write in place like the reference's ``(a, b, c, n)`` signatures do.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import raw


def _binary(a, b, op, out=None):
    if isinstance(b, torch.Tensor) and a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == a.dtype and a.shape == b.shape \
            and a.is_contiguous() and b.is_contiguous():
        r = raw.binary(a, b, op)
    else:
        r = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[op](a, b)
    if out is not None:
        out.copy_(r)
        return out
    return r


def add(a, b, out=None): return _binary(a, b, "add", out)
def sub(a, b, out=None): return _binary(a, b, "sub", out)
def mul(a, b, out=None): return _binary(a, b, "mul", out)
def div(a, b, out=None): return _binary(a, b, "div", out)
def fmadd(a, b, c): return torch.addcmul(c, a, b)                 # a*b + c
def fmsub(a, b, c): return a * b - c                              # a*b - c
def fnmadd(a, b, c): return torch.addcmul(c, a, b, value=-1)      # -(a*b) + c
def add_scalar(a, s): return a + s
def sub_scalar(a, s): return a - s
def mul_scalar(a, s): return a * s
def div_scalar(a, s): return a / s
def sub_mul_scalar(a, b, s): return (a - b) * s
def mul_add_scalar(a, m, s): return a * m + s
def set_scalar(a, s): return a.fill_(s)
def zero(a): return a.zero_()
def axpy(alpha, x, y): return y.add_(x, alpha=alpha)             # y += alpha * x (in place, like cublasAxpyEx)
def sqrt(a): return torch.sqrt(a)
def rsqrt(a): return torch.rsqrt(a)
def rcp(a): return torch.reciprocal(a)
def abs(a): return torch.abs(a)                                   # noqa: A001 - the reference's name
def min(a, b): return torch.minimum(a, b)                         # noqa: A001
def max(a, b): return torch.maximum(a, b)                         # noqa: A001
def scalar_max(a, s): return torch.clamp_min(a, s)
def clamp(a, lo, hi): return torch.clamp(a, lo, hi)
def equal(a, b): return (a == b).to(a.dtype)
def greater(a, b): return (a > b).to(a.dtype)
def copy(src, dst): return dst.copy_(src)
def cd_copy(src, dst): return dst.copy_(src, non_blocking=True)   # cross-device copy (ops.hpp:572-600)
def sum(a): return a.float().sum()                                # noqa: A001
def dot_product(a, b): return (a.float() * b.float()).sum()
def norm_squared(a): return a.float().pow(2).sum()
def sum_squared_diff(a, mean): return (a.float() - mean).pow(2).sum()
def cast(a, dtype): return a.to(dtype)


def bswap(a: torch.Tensor) -> torch.Tensor:
    """Byte-swap every element (endianness conversion of a received buffer)."""
    n = a.element_size()
    if n == 1:
        return a.clone()
    return a.contiguous().view(torch.uint8).view(-1, n).flip(1).contiguous().view(a.dtype).view(a.shape)


def fill_random_uniform(a: torch.Tensor, lo: float = 0.0, hi: float = 1.0, seed: Optional[int] = None) -> torch.Tensor:
    g = None if seed is None else torch.Generator(device=a.device).manual_seed(seed)
    return a.uniform_(lo, hi, generator=g)


def fill_random_normal(a: torch.Tensor, mean: float = 0.0, std: float = 1.0, seed: Optional[int] = None) -> torch.Tensor:
    g = None if seed is None else torch.Generator(device=a.device).manual_seed(seed)
    return a.normal_(mean, std, generator=g)


def check_equals(a: torch.Tensor, b: torch.Tensor, tol: float = 0.0) -> bool:
    return bool(torch.allclose(a.float(), b.float(), atol=tol, rtol=0.0))
