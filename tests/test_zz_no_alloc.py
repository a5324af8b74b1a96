"""The allocation-free batch-norm forward (``tnnb_batchnorm_fwd_noalloc``) against the regular entry point.

The file name sorts last on purpose: the built-in scratch array is per device and shared by every call,
so this test must hold both when it runs alone and after every other GPU test has used the library.
The exported C symbol is called directly through ctypes, the way a host without PyTorch would.
"""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from tnn_b200.ops import _lib

    lib = _lib.load()
    fn = lib.tnnb_batchnorm_fwd_noalloc
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, ci, cf, cf, ci, vp]
    fn.restype = ci
    lib.tnnb_noalloc_strerror.argtypes = [ci]
    lib.tnnb_noalloc_strerror.restype = ctypes.c_char_p
    lib.tnnb_batchnorm_noalloc_max_channels.argtypes = []
    lib.tnnb_batchnorm_noalloc_max_channels.restype = ci
    return lib


def _call(lib, x, y, gamma, beta, mean, rstd, rm, rv, eps, mom, relu):
    C = x.shape[-1]
    M = x.numel() // C
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.tnnb_batchnorm_fwd_noalloc(p(x), p(y), p(gamma), p(beta), p(mean), p(rstd), p(rm), p(rv), M, C, eps, mom, int(relu),
                                          stream)


@pytest.mark.parametrize("shape,relu,affine", [((32, 14, 14, 256), True, True), ((7, 5, 5, 64), False, True),
                                               ((64, 8, 8, 2048), True, False)])
def test_noalloc_matches_regular_twice(shape, relu, affine):
    from tnn_b200.ops import norm

    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    C = shape[-1]
    eps, mom = 1e-5, 0.1
    gamma = (torch.rand(C, device=dev) + 0.5).bfloat16() if affine else None
    beta = torch.randn(C, device=dev).bfloat16() if affine else None
    # two calls in a row with different inputs: the second must not see the sums of the first
    rm_a, rv_a = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    rm_b, rv_b = rm_a.clone(), rv_a.clone()
    for it in range(2):
        x = (torch.randn(shape, device=dev) * (1.5 + it) + 0.3 * it).bfloat16()
        y_ref, mean_ref, rstd_ref = norm.batchnorm_fwd_train(x, gamma, beta, rm_a, rv_a, eps, mom, relu)
        y = torch.empty_like(x)
        mean = torch.empty(C, dtype=torch.float32, device=dev)
        rstd = torch.empty_like(mean)
        gc.collect()  # garbage of earlier tests must not be freed between the two readings
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()   # what the driver has left: sees cudaMalloc calls of any origin
        rc = _call(lib, x, y, gamma, beta, mean, rstd, rm_b, rv_b, eps, mom, relu)
        assert rc == 0, lib.tnnb_noalloc_strerror(rc).decode()
        assert torch.cuda.memory_allocated() <= before  # the call took nothing from the tensor allocator
        torch.cuda.synchronize()
        if it > 0:  # the first call on a device may load the module that holds the scratch array (set-up)
            assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated behind the allocator's back"
        torch.cuda.synchronize()
        # plain fp32 reference of the same op
        x2 = x.float().reshape(-1, C)
        m = x2.mean(0)
        v = x2.var(0, unbiased=False)
        yy = (x2 - m) * torch.rsqrt(v + eps)
        if affine:
            yy = yy * gamma.float() + beta.float()
        if relu:
            yy = torch.relu(yy)
        assert torch.allclose(y.float().reshape(-1, C), yy, atol=3e-2, rtol=2e-2)
        assert torch.allclose(mean, m, atol=1e-3, rtol=1e-3)
        # and the regular entry point (same kernels; fp64 atomics may differ in the last bit)
        assert torch.allclose(y.float(), y_ref.float(), atol=2e-2, rtol=1e-2)
        assert torch.allclose(mean, mean_ref, atol=1e-5, rtol=1e-5)
        assert torch.allclose(rstd, rstd_ref, atol=1e-4, rtol=1e-4)
        assert torch.allclose(rm_b, rm_a, atol=1e-5, rtol=1e-5)
        assert torch.allclose(rv_b, rv_a, atol=1e-4, rtol=1e-4)


def test_noalloc_rejects_too_many_channels():
    lib = _lib()
    dev = torch.device("cuda", 0)
    cmax = lib.tnnb_batchnorm_noalloc_max_channels()
    assert cmax == 4096
    C = cmax + 8
    x = torch.zeros(4, C, device=dev, dtype=torch.bfloat16)
    y = torch.full_like(x, 7.0)
    f = lambda: torch.zeros(C, device=dev)
    rc = _call(lib, x, y, None, None, f(), f(), f(), f(), 1e-5, 0.1, False)
    assert rc == -2
    assert b"exceeds" in lib.tnnb_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float(y.float().min()) == 7.0  # nothing was launched
