"""Losses (reference: include/nn/loss.hpp:67-193,453-508).

``compute(logits, targets)`` returns ``(loss, grad)`` in one call: the cross-entropy kernel makes
both in a single pass over the logits and never synchronises with the host (the reference runs a
loss kernel, a two-stage reduction, a blocking copy of the scalar and a separate gradient kernel).
``loss`` is a 1-element device tensor; ``grad`` already includes ``scale`` (the ``1/accum`` or
``1/(microbatches*accum)`` factor of src/nn/train.cpp:284-286, coordinator.hpp:225).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import raw


class Loss:
    TYPE = "loss"

    def compute(self, pred: torch.Tensor, target: torch.Tensor, scale: float = 1.0, want_grad: bool = True
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError

    def corrects(self) -> Optional[torch.Tensor]:
        return None


class CrossEntropyLoss(Loss):
    """Softmax cross-entropy on logits, integer class labels, mean over rows (all dims but the last)."""
    TYPE = "crossentropy"

    def __init__(self, use_logits: bool = True):
        self.use_logits = use_logits
        self._corr = None

    def compute(self, pred, target, scale: float = 1.0, want_grad: bool = True, in_place: bool = False):
        V = pred.shape[-1]
        p2 = pred.reshape(-1, V)
        rows = p2.shape[0]
        if not self.use_logits:  # probabilities in: -log p[label]
            p = p2.float().clamp_min(1e-12)
            idx = target.reshape(-1).long()
            loss = -(p.gather(1, idx[:, None]).log()).mean().reshape(1)
            self._corr = (p.argmax(1) == idx).sum().to(torch.int32).reshape(1)
            grad = None
            if want_grad:
                grad = torch.zeros_like(p)
                grad.scatter_(1, idx[:, None], -1.0 / p.gather(1, idx[:, None]))
                grad = (grad * (scale / rows)).to(pred.dtype).reshape(pred.shape)
            return loss, grad
        loss, corr, grad = raw.softmax_ce(p2, target, V, (scale / rows) if want_grad else None, 1.0 / rows,
                                          grad_out=p2 if (in_place and want_grad) else None)
        self._corr = corr
        return loss, (grad.reshape(pred.shape) if grad is not None else None)

    def corrects(self):
        return self._corr


class _Regression(Loss):
    def _lg(self, d: torch.Tensor):
        raise NotImplementedError

    def compute(self, pred, target, scale: float = 1.0, want_grad: bool = True):
        d = pred.float() - target.float().reshape(pred.shape)
        l, g = self._lg(d)
        n = d.numel()
        loss = (l.sum() / n).reshape(1)
        grad = (g * (scale / n)).to(pred.dtype) if want_grad else None
        return loss, grad


class MSELoss(_Regression):
    TYPE = "mse"

    def _lg(self, d):
        return d * d, 2 * d


class MAELoss(_Regression):
    TYPE = "mae"

    def _lg(self, d):
        return d.abs(), torch.sign(d)


class HuberLoss(_Regression):
    TYPE = "huber"

    def __init__(self, delta: float = 1.0):
        self.delta = float(delta)

    def _lg(self, d):
        a = d.abs()
        quad = a <= self.delta
        return (torch.where(quad, 0.5 * d * d, self.delta * (a - 0.5 * self.delta)),
                torch.where(quad, d, self.delta * torch.sign(d)))


def create_loss(cfg: Optional[dict]) -> Loss:
    cfg = dict(cfg or {})
    t = str(cfg.get("type", "crossentropy")).lower()
    if t in ("crossentropy", "ce"):
        return CrossEntropyLoss(bool(cfg.get("use_logits", True)))
    if t in ("logsoftmax_crossentropy", "logsoftmax_ce"):
        return CrossEntropyLoss(True)
    if t == "mse":
        return MSELoss()
    if t == "mae":
        return MAELoss()
    if t == "huber":
        return HuberLoss(float(cfg.get("delta", 1.0)))
    raise ValueError(f"unknown loss type {t!r}")
