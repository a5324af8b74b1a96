"""Optimizers over a graph's flat buffers (reference: include/nn/optimizers.hpp:77-252).

One launch updates every parameter of the graph: the kernels read the flat fp32 gradient buffer,
update the fp32 master weights and the optimizer state, and write the bf16 compute copy in the
same pass (the reference launches one kernel per tensor and has no master copy). Non-trainable
entries of the flat buffer (batch-norm running statistics) are protected by keeping their
gradient at zero *and* by restoring them after weight decay. State can be saved and restored
(the reference checkpoints weights only).
"""
from __future__ import annotations

from typing import Dict, Optional

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
        self._hyper_host = torch.zeros(4, dtype=torch.float32).pin_memory() if dev.type == "cuda" else torch.zeros(4)

    def _push_hyper(self, lr, bc1, bc2, gscale):
        self._hyper_host[0], self._hyper_host[1], self._hyper_host[2], self._hyper_host[3] = lr, bc1, bc2, gscale
        self.hyper.copy_(self._hyper_host, non_blocking=True)

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
