"""Optimizers over a graph's flat buffers (reference: include/nn/optimizers.hpp:77-252).

One launch updates every parameter of the graph: the kernels read the flat fp32 gradient buffer,
update the fp32 master weights and the optimizer state, and write the bf16 compute copy in the
same pass (the reference launches one kernel per tensor and has no master copy). Non-trainable
entries of the flat buffer (batch-norm running statistics) are protected by keeping their
gradient at zero *and* by restoring them after weight decay. State can be saved and restored
(the reference checkpoints weights only).
"""
from __future__ import annotations

import os

from typing import List, Sequence,  Dict, Optional

import torch

from ..ops import raw


class Optimizer:
    TYPE = "optimizer"

    def __init__(self, learning_rate: float = 1e-3):
        self.lr = float(learning_rate)
        self.graph = None
        self.step_count = 0
        self.grad_scale = 1.0
        self.hyper: Optional[torch.Tensor] = None  # device copy of (lr, bc1, bc2, gscale) for CUDA-graph replay

    def attach(self, graph) -> "Optimizer":
        self.graph = graph
        self._alloc_state(graph.master_flat)
        # indices of non-trainable entries, found once here so that update() never synchronises
        idx = (~graph.trainable_mask).nonzero().squeeze(1)
        used = torch.zeros_like(graph.trainable_mask)
        for sl in graph.layer_slices.values():
            for (o, n, _, _) in sl:
                used[o:o + n] = True
        idx = (used & ~graph.trainable_mask).nonzero().squeeze(1)
        self._frozen_idx = idx if idx.numel() else None
        return self

    def _alloc_state(self, like: torch.Tensor) -> None:
        pass

    def get_learning_rate(self) -> float:
        return self.lr

    def set_learning_rate(self, lr: float) -> None:
        self.lr = float(lr)

    def enable_device_hyper(self) -> None:
        """Keep lr / bias corrections in device memory so a captured step sees new values."""
        dev = self.graph.master_flat.device
        self.hyper = torch.zeros(4, dtype=torch.float32, device=dev)
        # The upload is an asynchronous copy from pinned memory, and a replayed step is a single launch, so the host
        # can run several steps ahead of the device: every step gets a staging buffer of its own out of a small ring,
        # and a buffer is rewritten only after the copy that last read it has completed (its event).
        cuda = dev.type == "cuda"
        self._hyper_ring = [torch.zeros(4, dtype=torch.float32).pin_memory() if cuda else torch.zeros(4) for _ in range(8 if cuda else 1)]
        self._hyper_events = [torch.cuda.Event() if cuda else None for _ in self._hyper_ring]
        self._hyper_used = [False] * len(self._hyper_ring)
        self._hyper_next = 0

    def _push_hyper(self, lr, bc1, bc2, gscale):
        k = self._hyper_next
        self._hyper_next = (k + 1) % len(self._hyper_ring)
        buf, ev = self._hyper_ring[k], self._hyper_events[k]
        if ev is not None and self._hyper_used[k]:
            ev.synchronize()
        buf[0], buf[1], buf[2], buf[3] = lr, bc1, bc2, gscale
        self.hyper.copy_(buf, non_blocking=True)
        if ev is not None:
            ev.record()
            self._hyper_used[k] = True

    def prepare_step(self) -> None:
        """Host-side part of ``update`` (step count, hyper-parameter upload); call before a graph replay."""
        self.step_count += 1

    def update(self, prepared: bool = False) -> None:
        raise NotImplementedError

    def _views(self, sl=None):
        g = self.graph
        lp = g.params_flat if g.master_flat is not g.params_flat else None
        if sl is None:
            return g.master_flat, lp, g.grads_flat
        return g.master_flat[sl], (lp[sl] if lp is not None else None), g.grads_flat[sl]

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"step": torch.tensor(self.step_count), "lr": torch.tensor(self.lr)}

    def load_state_dict(self, d) -> None:
        self.step_count = int(d["step"])
        self.lr = float(d["lr"])


class SGD(Optimizer):
    """``p -= lr*g`` or, with momentum, ``v = mu*v - lr*g; p += v`` (sgd_kernels.cu:16-35)."""
    TYPE = "sgd"

    def __init__(self, learning_rate: float = 0.01, momentum: float = 0.0):
        super().__init__(learning_rate)
        self.momentum = float(momentum)
        self.velocity: Optional[torch.Tensor] = None

    def _alloc_state(self, like):
        self.velocity = torch.zeros_like(like) if self.momentum != 0.0 else None

    def prepare_step(self):
        super().prepare_step()
        if self.hyper is not None:
            self._push_hyper(self.lr, 1.0, 1.0, self.grad_scale)

    def update(self, prepared: bool = False, sl=None):
        if not prepared:
            self.prepare_step()
        m, lp, g = self._views(sl)
        v = self.velocity if (sl is None or self.velocity is None) else self.velocity[sl]
        raw.sgd_step(m, lp, g, v, self.lr, self.momentum, self.grad_scale, self.hyper)

    def state_dict(self):
        d = super().state_dict()
        if self.velocity is not None:
            d["velocity"] = self.velocity
        return d

    def load_state_dict(self, d):
        super().load_state_dict(d)
        if "velocity" in d and self.velocity is not None:
            self.velocity.copy_(d["velocity"])


class Adam(Optimizer):
    """Adam with bias correction; both weight-decay modes apply ``p -= wd*lr*p`` like the reference
    (adam_kernels.cu:28-53), so ``decouple_weight_decay`` only changes the reported name."""
    TYPE = "adam"

    def __init__(self, learning_rate: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8,
                 weight_decay: float = 0.0, decouple_weight_decay: bool = False):
        super().__init__(learning_rate)
        self.beta1, self.beta2, self.eps, self.weight_decay = float(beta1), float(beta2), float(epsilon), float(weight_decay)
        self.decoupled = bool(decouple_weight_decay)
        self.m: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None

    def _alloc_state(self, like):
        self.m, self.v = torch.zeros_like(like), torch.zeros_like(like)

    def prepare_step(self):
        super().prepare_step()
        if self.hyper is not None:
            self._push_hyper(self.lr, 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count, self.grad_scale)

    def update(self, prepared: bool = False, sl=None):
        if not prepared:
            self.prepare_step()
        g = self.graph
        frozen = None
        if self.weight_decay != 0.0 and self._frozen_idx is not None and sl is None:
            frozen = g.master_flat.index_select(0, self._frozen_idx)
        m, lp, gr = self._views(sl)
        mm, vv = (self.m, self.v) if sl is None else (self.m[sl], self.v[sl])
        raw.adam_step(m, lp, gr, mm, vv, self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.step_count,
                      self.grad_scale, self.hyper)
        if frozen is not None:  # weight decay must not touch batch-norm running statistics
            g.master_flat.index_copy_(0, self._frozen_idx, frozen)
            if g.master_flat is not g.params_flat:
                g.params_flat.index_copy_(0, self._frozen_idx, frozen.to(g.params_flat.dtype))

    def state_dict(self):
        d = super().state_dict()
        d.update(m=self.m, v=self.v)
        return d

    def load_state_dict(self, d):
        super().load_state_dict(d)
        self.m.copy_(d["m"])
        self.v.copy_(d["v"])


class AdamW(Adam):
    TYPE = "adamw"

    def __init__(self, learning_rate: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8,
                 weight_decay: float = 0.01, **_):
        super().__init__(learning_rate, beta1, beta2, epsilon, weight_decay, True)


def plan_buckets(points: Sequence[int], lo: int, hi: int, n_buckets: int, min_bucket: int) -> List[tuple]:
    """Cut ``[lo, hi)`` into buckets ``(lo_i, hi_i)`` in the order backward finishes them (highest offsets first).
    ``points`` are the offsets ``Graph.grad_hook`` reports, in firing order; a bucket ends at such a point and holds
    at least ``max(min_bucket, (hi - lo) / n_buckets)`` elements (the last one takes what is left)."""
    target = max(min_bucket, (hi - lo) // max(1, n_buckets))
    out, top = [], hi
    for pt in points:
        pt = pt // 8 * 8
        if lo < pt < top and top - pt >= target:
            out.append((pt, top))
            top = pt
    out.append((lo, top))
    return out


class OverlappedUpdate:
    """The optimizer step of a single-GPU job, spread under the backward pass.

    The update is memory bound and small in registers; backward is a chain of tensor-core kernels. The flat parameter
    buffer is laid out in first-use order, so backward finishes its gradients from the end: the buffer is cut into
    buckets in that order (:func:`plan_buckets`) and a bucket's update (followed by the clearing of its gradients) is
    launched on a second stream as soon as ``Graph.grad_hook`` reports its gradients final, while backward goes on in
    the main stream. Only the last bucket (the embeddings) runs after backward. A bucket's parameters are no longer read
    by the backward pass in progress, and ``update`` joins the second stream before the next forward pass.
    The data-parallel optimizer does the same with its reduce + update + broadcast kernel (``parallel/dp.py``).

    Wraps an :class:`Optimizer` and offers its surface; ``clears_grads`` tells the trainer that the gradient slab is
    already zero after ``update``."""

    clears_grads = True

    def __init__(self, opt: Optimizer, graph, n_buckets: int = 4, min_bucket: int = 4 << 20):
        self.opt, self.graph = opt, graph
        min_bucket = int(os.environ.get("TNNB_UPDATE_MIN_BUCKET", str(min_bucket)))  # tests lower it for tiny models
        self.spans = plan_buckets(graph.grad_ready_points(), 0, graph.total_elems, n_buckets, min_bucket)
        self.side = torch.cuda.Stream(device=graph.master_flat.device, priority=-1)
        self._next = 0
        self._prepared = False
        graph.grad_hook = self._on_grads_ready

    @staticmethod
    def usable(opt: Optimizer, graph) -> bool:
        """Needs a CUDA graph whose gradients become final in buffer order, and no entries that a decaying update
        must skip (the sliced update does not put batch-norm running statistics back)."""
        if graph.master_flat is None or graph.master_flat.device.type != "cuda" or not graph.grad_hook_usable():
            return False
        if getattr(opt, "weight_decay", 0.0) != 0.0 and getattr(opt, "_frozen_idx", None) is not None:
            return False
        return graph.grad_hook is None

    # ---- the optimizer's surface
    def __getattr__(self, name):  # lr, hyper, state_dict, ... of the wrapped optimizer
        return getattr(self.__dict__["opt"], name)

    @property
    def step_count(self):
        return self.opt.step_count

    @step_count.setter
    def step_count(self, v):
        self.opt.step_count = v

    def prepare_step(self):
        self.opt.prepare_step()
        self._prepared = True

    def _bucket(self, lo: int, hi: int):
        self.opt.update(prepared=True, sl=slice(lo, hi))
        self.graph.grads_flat[lo:hi].zero_()

    def _on_grads_ready(self, floor: int):
        """``Graph.grad_hook``: every gradient at a flat offset >= ``floor`` is final."""
        if not self.graph.training:
            return
        upto = self._next
        while upto < len(self.spans) - 1 and self.spans[upto][0] >= floor:  # the last bucket goes with update()
            upto += 1
        if upto == self._next:
            return
        if not self._prepared:
            self.prepare_step()
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            while self._next < upto:
                self._bucket(*self.spans[self._next])
                self._next += 1

    def update(self, prepared: bool = False):
        if prepared:
            self._prepared = True
        if not self._prepared:
            self.prepare_step()
        while self._next < len(self.spans):  # what backward did not release early, at least the last bucket
            self._bucket(*self.spans[self._next])
            self._next += 1
        ev = torch.cuda.Event()
        ev.record(self.side)
        torch.cuda.current_stream().wait_event(ev)
        self._next = 0
        self._prepared = False


def create_optimizer(cfg: Optional[dict]) -> Optimizer:
    """Factory from ``{"type": "adam"|"adamw"|"sgd", ...}`` (src/nn/train.cpp:57-72 copies the keys)."""
    cfg = dict(cfg or {})
    t = str(cfg.get("type", "adam")).lower()
    lr = float(cfg.get("learning_rate", cfg.get("lr", 1e-3)))
    if t == "sgd":
        return SGD(lr, float(cfg.get("momentum", 0.0)))
    kw = dict(beta1=float(cfg.get("beta1", 0.9)), beta2=float(cfg.get("beta2", 0.999)), epsilon=float(cfg.get("epsilon", 1e-8)),
              weight_decay=float(cfg.get("weight_decay", 0.0)))
    if t == "adamw":
        return AdamW(lr, **kw)
    if t == "adam":
        return Adam(lr, decouple_weight_decay=bool(cfg.get("decouple_weight_decay", False)), **kw)
    raise ValueError(f"unknown optimizer type {t!r}")
