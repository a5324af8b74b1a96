"""Data-parallel optimizer step.

``FusedDPOptimizer`` runs the hand-written kernel ``tnnb_dp_step`` (csrc/kernels/comm_fused.cu):
gradient reduce-scatter over NVLink peer loads, 1/N scale, AdamW / SGD-momentum on the rank's
fp32 master slice (optimizer state is sharded, ZeRO-1 style) and parameter all-gather by peer
stores, all in one launch per region. ``NcclDPOptimizer`` does the same with
``reduce_scatter_tensor`` / ``all_gather_into_tensor`` around the local update kernel - the
"only calls NCCL" baseline - and also serves gloo/CPU tests with an all-reduce.

A *region* is a range of the flat buffers together with the ranks that hold a replica of it: with
tensor parallelism the replicated parameters (embeddings, layernorms, head) are reduced over
every rank of the job and the sharded ones only over the data-parallel group. The reference has
no data parallelism to compare with (include/distributed/coordinator.hpp:618-620 is a stub).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..nn.optim import SGD, Adam, Optimizer, plan_buckets  # noqa: F401 (re-exported: tests and callers import it from here)
from ..ops import _lib
from ..ops.gemm import LAUNCHES
from .symm import SymmetricHeap, ptr_array


@dataclass
class Region:
    lo: int
    hi: int
    ranks: List[int]          # global ranks that replicate this range (this rank included)
    group: Optional[object] = None  # matching torch.distributed group (NCCL baseline)


def _declare(lib):
    vp, ll, f, i, u = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_int, ctypes.c_uint
    lib.tnnb_dp_step.argtypes = [i, i, vp, vp, vp, vp, vp, vp, vp, ll, ll, i, f, f, f, f, f, f, f, f, f, vp, u, vp, vp, vp, vp, vp]
    lib.tnnb_dp_step.restype = i


class FusedDPOptimizer:
    """Drives ``tnnb_dp_step`` for every region of a graph whose flat buffers live in ``heap``.

    ``overlap=True`` (pure data parallelism, one region over the whole buffer, one backward pass per step) cuts the
    region into buckets that follow the order in which backward finishes the gradients - the flat buffer is laid out
    in first-use order, so backward completes it from the end - and starts a bucket's reduce + update + broadcast
    kernel on a second stream as soon as ``Graph.grad_hook`` reports its gradients final, while backward keeps
    running on the main stream. Only the last bucket (the embeddings, finished at the very end) is exposed."""

    MIN_BUCKET = 4 << 20  # elements

    def __init__(self, opt: Optimizer, graph, heap: SymmetricHeap, regions: Sequence[Region], grad_scale: float,
                 overlap: bool = False, n_buckets: int = 4):
        self.opt, self.graph, self.heap, self.regions = opt, graph, heap, list(regions)
        self.lib = _lib.load()
        _declare(self.lib)
        opt.graph = graph
        opt.grad_scale = grad_scale
        self.me = dist.get_rank() if dist.is_initialized() else 0
        dev = graph.master_flat.device
        self.is_adam = isinstance(opt, Adam)
        # number of updates so far, kept on the device so that a captured CUDA graph advances it on replay
        self.tick = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overlap = bool(overlap and len(self.regions) == 1 and len(self.regions[0].ranks) > 1
                            and self.regions[0].lo == 0 and self.regions[0].hi == graph.total_elems and graph.grad_hook_usable())
        spans = []  # (lo, hi, region) in launch order
        if self.overlap:
            reg = self.regions[0]
            min_bucket = int(os.environ.get("TNNB_DP_MIN_BUCKET", str(self.MIN_BUCKET)))  # tests lower it for tiny models
            spans = [(a, b, reg) for a, b in plan_buckets(graph.grad_ready_points(), reg.lo, reg.hi, n_buckets, min_bucket)]
            self.overlap = len(spans) > 1
        else:
            spans = [(reg.lo, reg.hi, reg) for reg in self.regions]
        self.sites = []
        for (blo, bhi, reg) in spans:
            n = len(reg.ranks)
            idx = reg.ranks.index(self.me)
            span = bhi - blo
            per = (span // n) // 8 * 8
            lo = blo + idx * per
            hi = bhi if idx == n - 1 else lo + per
            flags = heap.alloc((16,), torch.int32).zero_()
            site = {
                "n": n, "idx": idx, "lo": lo, "hi": hi, "epoch": 0, "bucket_lo": blo, "bucket_hi": bhi,
                "flags": ptr_array(heap.peer_ptrs(flags, reg.ranks)),
                "grads": ptr_array(heap.peer_ptrs(graph.grads_flat, reg.ranks)),
                "lp": ptr_array(heap.peer_ptrs(graph.params_flat, reg.ranks)) if graph.master_flat is not graph.params_flat else None,
                "f32": ptr_array(heap.peer_ptrs(graph.params_flat, reg.ranks)) if graph.master_flat is graph.params_flat else None,
                "m": torch.zeros(max(hi - lo, 8), dtype=torch.float32, device=dev),
                "v": torch.zeros(max(hi - lo, 8), dtype=torch.float32, device=dev) if self.is_adam else None,
                "go": torch.zeros(1, dtype=torch.int32, device=dev), "done": torch.zeros(1, dtype=torch.int32, device=dev),
            }
            self.sites.append(site)
        # Entries that are stored as parameters but never trained (batch-norm running statistics): weight decay
        # must not shrink them, so their values are put back after a decaying update (indices found once here).
        used = torch.zeros_like(graph.trainable_mask)
        for sl in graph.layer_slices.values():
            for ent in sl:
                if ent:
                    used[ent[0]:ent[0] + ent[1]] = True
        idx = (used & ~graph.trainable_mask).nonzero().squeeze(1)
        self._frozen_idx = idx if idx.numel() else None
        # per-step state of the overlapped launch sequence
        self._prepared = False   # opt.prepare_step() done for the step in progress
        self._begun = False      # tick advanced / arguments computed for the step in progress
        self._next = 0           # next site to launch
        self._args = None
        self._frozen = None
        self.comm = torch.cuda.Stream(device=dev, priority=-1) if self.overlap else None
        if self.overlap:
            graph.grad_hook = self._on_grads_ready
        # a parameter written by a peer lands in params_flat; when params are fp32 the master *is* params_flat
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()

    # Optimizer-compatible surface used by the trainer
    def get_learning_rate(self):
        return self.opt.get_learning_rate()

    def set_learning_rate(self, lr):
        self.opt.set_learning_rate(lr)

    def enable_device_hyper(self):
        self.opt.enable_device_hyper()

    def prepare_step(self):
        self.opt.prepare_step()
        self._prepared = True

    @property
    def hyper(self):
        return self.opt.hyper

    @property
    def step_count(self):
        return self.opt.step_count

    @step_count.setter
    def step_count(self, v):
        self.opt.step_count = v

    # ------------------------------------------------------------------ one step = begin, launches, finish
    def _begin(self):
        """First launch of a step: advance the step count and the device tick, fix the kernel arguments."""
        if self._begun:
            return
        o, g = self.opt, self.graph
        if not self._prepared:
            self.prepare_step()
        if self.is_adam:
            bc1, bc2 = 1 - o.beta1 ** o.step_count, 1 - o.beta2 ** o.step_count
            self._args = (0, o.lr, o.beta1, o.beta2, o.eps, o.weight_decay, bc1, bc2, o.grad_scale, 0.0)
        else:
            self._args = (1, o.lr, 0.0, 0.0, 0.0, 0.0, 1.0, 1.0, o.grad_scale, o.momentum)
        self._frozen = None
        if self.is_adam and o.weight_decay != 0.0 and self._frozen_idx is not None:
            self._frozen = g.master_flat.index_select(0, self._frozen_idx)
        self.tick.add_(1)
        self._next = 0
        self._begun = True

    def _launch(self, s):
        o, g, args = self.opt, self.graph, self._args
        status = _lib.ptr(_lib.status_word(g.master_flat.device))
        rc = self.lib.tnnb_dp_step(
            s["n"], s["idx"], s["flags"], s["grads"], s["lp"], s["f32"], _lib.ptr(g.master_flat), _lib.ptr(s["m"]),
            _lib.ptr(s["v"]), s["lo"], s["hi"], args[0], args[1], args[2], args[3], args[4], args[5], args[6], args[7],
            args[8], args[9], _lib.ptr(o.hyper), 0, _lib.ptr(self.tick), _lib.ptr(s["go"]), _lib.ptr(s["done"]), status,
            _lib.stream())
        _lib.check_rc(rc, "tnnb_dp_step")
        LAUNCHES["count"] += 1

    def _launch_on_comm(self, upto: int):
        """Launch sites ``[_next, upto)`` on the communication stream, ordered after everything queued so far."""
        if upto <= self._next:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.comm.wait_event(ev)
        with torch.cuda.stream(self.comm):
            while self._next < upto:
                self._launch(self.sites[self._next])
                self._next += 1

    def _on_grads_ready(self, floor: int):
        """``Graph.grad_hook``: every gradient at a flat offset >= ``floor`` is final."""
        if not self.overlap or not self.graph.training:
            return
        upto = self._next if self._begun else 0
        while upto < len(self.sites) - 1 and self.sites[upto]["bucket_lo"] >= floor:  # the last bucket goes with update()
            upto += 1
        if upto > (self._next if self._begun else 0):
            self._begin()
            self._launch_on_comm(upto)

    def update(self, prepared: bool = False):
        if prepared:
            self._prepared = True
        self._begin()
        g = self.graph
        if self.overlap:
            self._launch_on_comm(len(self.sites))
            ev = torch.cuda.Event()
            ev.record(self.comm)
            torch.cuda.current_stream().wait_event(ev)
        else:
            while self._next < len(self.sites):
                self._launch(self.sites[self._next])
                self._next += 1
        if self._frozen is not None:  # the kernel returns only after every peer's writes into this rank have landed
            g.master_flat.index_copy_(0, self._frozen_idx, self._frozen)
            if g.params_flat is not g.master_flat:
                g.params_flat.index_copy_(0, self._frozen_idx, self._frozen.to(g.params_flat.dtype))
            self._frozen = None
        self._prepared = self._begun = False

    def state_dict(self):
        d = self.opt.state_dict()
        for k, s in enumerate(self.sites):
            d[f"m{k}"] = s["m"]
            if s["v"] is not None:
                d[f"v{k}"] = s["v"]
        return d

    def load_state_dict(self, d):
        self.opt.step_count = int(d["step"])
        self.opt.lr = float(d["lr"])
        for k, s in enumerate(self.sites):
            s["m"].copy_(d[f"m{k}"])
            if s["v"] is not None:
                s["v"].copy_(d[f"v{k}"])

    # --- the unsharded form of the state: what a single-process optimizer of the same type saves and loads ---
    def full_state(self, group=None) -> dict:
        """Moments gathered to full-length flat vectors (``m``/``v`` for Adam, ``velocity`` for SGD) plus the
        fp32 master values of every slice from the rank that owns them. Collective over ``group`` (the ranks that
        share the slices); every rank gets the result. Only meaningful when one region covers the whole buffer."""
        g = self.graph
        n = g.total_elems
        dev = g.master_flat.device
        full_m = torch.zeros(n, dtype=torch.float32, device=dev)
        full_v = torch.zeros(n, dtype=torch.float32, device=dev) if self.is_adam else None
        master = torch.zeros(n, dtype=torch.float32, device=dev)
        for s in self.sites:
            lo, hi = s["lo"], s["hi"]
            full_m[lo:hi] = s["m"][:hi - lo]
            if full_v is not None:
                full_v[lo:hi] = s["v"][:hi - lo]
            master[lo:hi] = g.master_flat[lo:hi]
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            for t in (full_m, full_v, master):
                if t is not None:
                    dist.all_reduce(t, group=group)
        d = {"step": torch.tensor(self.opt.step_count), "lr": torch.tensor(self.opt.lr), "master": master}
        if self.is_adam:
            d.update(m=full_m, v=full_v)
        else:
            d["velocity"] = full_m
        return d

    def load_full_state(self, d) -> None:
        """Inverse of :meth:`full_state` for this rank's slices; ``d`` may come from a single-process optimizer."""
        self.opt.step_count = int(d["step"])
        self.opt.lr = float(d["lr"])
        first = d.get("m", d.get("velocity"))
        for s in self.sites:
            lo, hi = s["lo"], s["hi"]
            if first is not None:
                s["m"][:hi - lo].copy_(first[lo:hi])
            if s["v"] is not None and "v" in d:
                s["v"][:hi - lo].copy_(d["v"][lo:hi])


class NcclDPOptimizer:
    """Library-collective version: all-reduce (gloo/CPU) or reduce-scatter + all-gather (NCCL) around
    the local update kernels. Used as the baseline of the fused path and on CPU."""

    def __init__(self, opt: Optimizer, graph, regions: Sequence[Region], grad_scale: float):
        self.opt, self.graph, self.regions = opt, graph, list(regions)
        opt.attach(graph)
        opt.grad_scale = grad_scale

    def __getattr__(self, name):
        return getattr(self.__dict__["opt"], name)

    @property
    def step_count(self):
        return self.opt.step_count

    @step_count.setter
    def step_count(self, v):
        self.opt.step_count = v

    def update(self, prepared: bool = False):
        g = self.graph
        for reg in self.regions:
            if len(reg.ranks) > 1:
                dist.all_reduce(g.grads_flat[reg.lo:reg.hi], group=reg.group)
        self.opt.update(prepared=prepared)
