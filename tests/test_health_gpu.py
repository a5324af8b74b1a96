"""Device side of failure detection: a bounded wait on a flag nothing sets returns a status code the host reads,
and the CUDA context stays usable afterwards."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_expires_with_status_and_context_survives():
    from tnn_b200.ops import _lib
    from tnn_b200.ops.gemm import gemm
    from tnn_b200.parallel.health import KernelTimeout, check_device_status

    lib = _lib.load()
    lib.tnnb_flag_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p]
    lib.tnnb_flag_set.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]
    dev = torch.device("cuda", 0)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    status = _lib.status_word(dev)
    _lib.check_status(dev)
    t0 = time.time()
    rc = lib.tnnb_flag_wait(_lib.ptr(flag), 1, 300_000_000, _lib.ptr(status), _lib.stream())  # 0.3 s, nothing sets the flag
    assert rc == 0
    torch.cuda.synchronize()
    assert 0.25 < time.time() - t0 < 5.0
    with pytest.raises(KernelTimeout):
        check_device_status(dev)
    check_device_status(dev)  # the status word was cleared by the failed check
    # the context is fine: a flag that is already set passes at once, and real work still runs
    assert lib.tnnb_flag_set(_lib.ptr(flag), 5, _lib.stream()) == 0
    torch.cuda.synchronize()
    t0 = time.time()
    assert lib.tnnb_flag_wait(_lib.ptr(flag), 5, 5_000_000_000, _lib.ptr(status), _lib.stream()) == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    check_device_status(dev)
    a = torch.randn(256, 128, device=dev).bfloat16()
    b = torch.randn(256, 128, device=dev).bfloat16()
    out = gemm(a, b)
    assert torch.allclose(out.float(), a.float() @ b.float().t(), atol=0.5, rtol=0.05)
