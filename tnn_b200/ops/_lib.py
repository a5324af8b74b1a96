"""ctypes binding of ``libtnnb_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`tnn_b200._build`. Every op in
:mod:`tnn_b200.ops` dispatches CUDA tensors to it and raises if it cannot be
loaded - there is no silent PyTorch fallback for tensors that live on a GPU.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_LOCK = threading.Lock()
_LIB = None
_STATUS = {}

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_ull = ctypes.c_ulonglong


def bounds_checked() -> bool:
    """True when this process runs the bounds-checked build of the kernels (``TNNB_BOUNDS_CHECK=1``)."""
    return os.environ.get("TNNB_BOUNDS_CHECK", "") == "1"


def lib_path() -> str:
    """``TNNB_KERNEL_LIB`` names another build of the kernel library to load (A/B comparisons of a kernel change)."""
    from .. import _build

    return os.environ.get("TNNB_KERNEL_LIB") or _build.kernels_path(bounds_checked())


def load(build_if_missing: bool = True):
    """Return the loaded kernel library (building it first if necessary)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not os.path.exists(path):
            if not build_if_missing:
                raise RuntimeError(f"tnn_b200 kernel library missing: {path}")
            from .. import _build

            _build.build_kernels(bounds_check=bounds_checked())
        lib = ctypes.CDLL(path)
        _declare(lib)
        _LIB = lib
    return _LIB


def _declare(lib):
    def sig(name, args, res=c_int):
        fn = getattr(lib, name, None)
        if fn is None:
            return
        fn.argtypes = args
        fn.restype = res

    sig("tnnb_gemm_bf16", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll,
                           c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int,
                           c_void_p, c_void_p])
    sig("tnnb_act_fwd", [c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p])
    sig("tnnb_act_bwd", [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p])
    sig("tnnb_binary", [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p])
    sig("tnnb_dropout", [c_void_p, c_void_p, c_ll, c_float, c_ull, c_void_p, c_void_p])
    sig("tnnb_embedding_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_ll, c_ll, c_float,
                               c_ull, c_void_p, c_void_p])
    sig("tnnb_embedding_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_ll, c_ll, c_float,
                               c_ull, c_void_p, c_void_p])
    sig("tnnb_colsum_accum", [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p])
    sig("tnnb_cast_f32_bf16", [c_void_p, c_void_p, c_ll, c_void_p])
    sig("tnnb_layernorm_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_ll, c_int, c_float, c_float, c_ull, c_void_p, c_void_p])
    sig("tnnb_layernorm_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_ll, c_int, c_float, c_ull, c_void_p, c_void_p])
    sig("tnnb_softmax_ce", [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int,
                            c_float, c_float, c_void_p])
    sig("tnnb_adam_step", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float,
                           c_float, c_float, c_float, c_float, c_float, c_void_p, c_void_p])
    sig("tnnb_sgd_step", [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_void_p,
                          c_void_p])
    sig("tnnb_attn_fwd", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                          c_void_p])
    sig("tnnb_attn_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_float, c_void_p, c_void_p])


def ptr(t):
    """Device/host address of a tensor (None -> NULL)."""
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write an error code into."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    w = _STATUS.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _STATUS[key] = w
    return w


_STATUS_NAMES = {
    0: "ok", 1: "timeout in TMA producer", 2: "timeout in MMA issuer", 3: "timeout in epilogue",
    4: "timeout waiting for a peer", 5: "bad argument",
}


def check_status(device=None):
    """Synchronise and raise if any kernel recorded a bounded-wait expiry since the last check."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"tnn_b200 kernel reported status {code}: {_STATUS_NAMES.get(code, '?')}")


_BOUNDS_FILES = ("elementwise", "loss_optim", "conv_pool", "batchnorm")


def fetch_bounds_violations():
    """Read and clear the bounds records of the checked build: a list of ``{"file", "line", "index", "limit"}`` (first
    violation per kernel source file). Synchronises the device. Raises if the loaded library is the regular build."""
    lib = load()
    out = []
    for name in _BOUNDS_FILES:
        fn = getattr(lib, "tnnb_bounds_fetch_" + name)
        fn.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_longlong)]
        fn.restype = ctypes.c_int
        hl = (ctypes.c_int * 2)()
        il = (ctypes.c_longlong * 2)()
        rc = fn(hl, il)
        if rc == -1:
            raise RuntimeError("the loaded kernel library is not the bounds-checked build (set TNNB_BOUNDS_CHECK=1 before importing)")
        if rc != 0:
            raise RuntimeError(f"reading the bounds record of {name} failed ({rc})")
        if hl[0]:
            out.append({"file": name + ".cu", "line": int(hl[1]), "index": int(il[0]), "limit": int(il[1])})
    return out


def check_bounds():
    """Raise ``IndexError`` if a kernel of the checked build recorded an out-of-range index since the last call."""
    v = fetch_bounds_violations()
    if v:
        raise IndexError("; ".join(f"{r['file']}:{r['line']} index {r['index']} outside [0, {r['limit']})" for r in v))


def check_rc(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} rejected the call (code {rc})")
