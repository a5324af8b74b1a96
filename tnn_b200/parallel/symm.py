"""Symmetric heap: one device slab per rank, exported to every other rank of the node with CUDA
IPC, sub-allocated identically on all ranks so that a buffer has the same offset everywhere.

It replaces the reference's ``IbvAllocator`` (a pinned host slab registered for RDMA,
include/device/ibv_allocator.hpp:31-160): here the slab is device memory reachable over NVLink
with plain loads and stores from SM code, which is what the fused compute+collective kernels
(csrc/kernels/comm_fused.cu) use. Sub-allocation is done by the C++ ``PoolAllocator`` of the host
runtime; the IPC handles travel through ``torch.distributed`` (any backend, gloo included).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..host import H
from ..ops import _lib

_DT = {torch.float32: ("<f4", 4), torch.bfloat16: ("<u2", 2), torch.int32: ("<i4", 4), torch.uint8: ("|u1", 1),
       torch.int64: ("<i8", 8)}


class _Raw:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can alias it."""

    def __init__(self, ptr: int, nbytes: int, typestr: str, itemsize: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // itemsize,), "typestr": typestr, "data": (ptr, False), "version": 2}


def tensor_at(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A torch tensor aliasing ``numel*itemsize`` bytes at device address ``ptr`` (no ownership)."""
    n = 1
    for s in shape:
        n *= int(s)
    typestr, item = _DT[dtype]
    flat = torch.as_tensor(_Raw(ptr, max(n, 1) * item, typestr, item), device=device)
    if dtype == torch.bfloat16:
        flat = flat.view(torch.bfloat16)
    return flat[:n].view(*shape)


class SymmetricHeap:
    """``heap = SymmetricHeap(nbytes, group)``; ``t = heap.alloc(shape, dtype)``; ``heap.peer_ptrs(t)``.

    All ranks of ``group`` must perform the same sequence of ``alloc`` calls. ``group`` may be
    ``None`` for a single process (the heap then behaves like a private slab).
    """

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.lib = _lib.load()
        self.lib.tnnb_symm_malloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_ulonglong]
        self.lib.tnnb_ipc_export.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        self.lib.tnnb_ipc_import.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
        self.lib.tnnb_ipc_close.argtypes = [ctypes.c_void_p]
        self.lib.tnnb_symm_free.argtypes = [ctypes.c_void_p]
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(nbytes)
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        base = ctypes.c_void_p()
        _lib.check_rc(self.lib.tnnb_symm_malloc(ctypes.byref(base), self.nbytes), "symmetric heap allocation")
        self.base = int(base.value)
        self.pool = H.PoolAllocator(self.nbytes, 256)
        self.peer_base: List[int] = [self.base] * self.world
        self._opened: List[int] = []
        if self.world > 1:
            handle = ctypes.create_string_buffer(64)
            _lib.check_rc(self.lib.tnnb_ipc_export(ctypes.c_void_p(self.base), handle), "cudaIpcGetMemHandle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                out = ctypes.c_void_p()
                buf = ctypes.create_string_buffer(h, 64)
                _lib.check_rc(self.lib.tnnb_ipc_import(buf, ctypes.byref(out)), "cudaIpcOpenMemHandle")
                self.peer_base[r] = int(out.value)
                self._opened.append(int(out.value))
            dist.barrier(group=group)

    def alloc(self, shape: Sequence[int], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        off = self.pool.allocate(max(n, 1) * _DT[dtype][1])
        if off < 0:
            raise MemoryError(f"symmetric heap exhausted ({self.nbytes} bytes)")
        t = tensor_at(self.base + off, shape, dtype, self.device)
        t._symm_offset = off  # noqa: SLF001 - remembered for peer address arithmetic
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor does not live in this symmetric heap")
        return off

    def peer_ptrs(self, t: torch.Tensor, ranks: Optional[Sequence[int]] = None) -> List[int]:
        """Device addresses of the same buffer on each rank (index = rank inside the heap's group)."""
        off = self.offset_of(t)
        ranks = range(self.world) if ranks is None else ranks
        return [self.peer_base[r] + off for r in ranks]

    def peer_view(self, t: torch.Tensor, rank: int) -> torch.Tensor:
        """A tensor aliasing rank ``rank``'s copy of ``t`` (debugging / tests; kernels use raw pointers)."""
        return tensor_at(self.peer_base[rank] + self.offset_of(t), t.shape, t.dtype, self.device)

    def close(self):
        for p in self._opened:
            self.lib.tnnb_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.base:
            torch.cuda.synchronize()
            self.lib.tnnb_symm_free(ctypes.c_void_p(self.base))
            self.base = 0


def ptr_array(ptrs: Sequence[Optional[int]]):
    """ctypes ``void*[n]`` from a list of addresses (None -> NULL)."""
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = ctypes.c_void_p(p) if p else None
    return arr
