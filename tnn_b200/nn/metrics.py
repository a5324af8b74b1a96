"""Evaluation metrics (reference: include/nn/metrics.hpp:164-314). Not on the training hot path:
the arg-max-correct count used during training comes out of the cross-entropy kernel."""
from __future__ import annotations

import math

import torch


def class_corrects(pred: torch.Tensor, labels: torch.Tensor) -> int:
    return int((pred.reshape(-1, pred.shape[-1]).float().argmax(1) == labels.reshape(-1).to(pred.device)).sum())


def accuracy(pred, labels) -> float:
    return class_corrects(pred, labels) / max(1, labels.numel())


def top_k_accuracy(pred, labels, k: int = 5) -> float:
    p = pred.reshape(-1, pred.shape[-1]).float()
    top = p.topk(min(k, p.shape[1]), 1).indices
    return float((top == labels.reshape(-1, 1).to(p.device)).any(1).float().mean())


def confusion_counts(pred, labels, num_classes: int):
    p = pred.reshape(-1, pred.shape[-1]).float().argmax(1).cpu()
    l = labels.reshape(-1).cpu().long()
    tp = torch.zeros(num_classes)
    fp = torch.zeros(num_classes)
    fn = torch.zeros(num_classes)
    for c in range(num_classes):
        tp[c] = ((p == c) & (l == c)).sum()
        fp[c] = ((p == c) & (l != c)).sum()
        fn[c] = ((p != c) & (l == c)).sum()
    return tp, fp, fn


def precision(pred, labels, num_classes: int, macro: bool = True):
    tp, fp, _ = confusion_counts(pred, labels, num_classes)
    per = tp / (tp + fp).clamp(min=1)
    return float(per.mean()) if macro else per


def recall(pred, labels, num_classes: int, macro: bool = True):
    tp, _, fn = confusion_counts(pred, labels, num_classes)
    per = tp / (tp + fn).clamp(min=1)
    return float(per.mean()) if macro else per


def f1_score(pred, labels, num_classes: int, macro: bool = True):
    tp, fp, fn = confusion_counts(pred, labels, num_classes)
    per = 2 * tp / (2 * tp + fp + fn).clamp(min=1)
    return float(per.mean()) if macro else per


def perplexity(mean_cross_entropy: float) -> float:
    return math.exp(min(mean_cross_entropy, 80.0))


def mae(pred, target) -> float:
    return float((pred.float() - target.float()).abs().mean())


def mse(pred, target) -> float:
    return float(((pred.float() - target.float()) ** 2).mean())


def rmse(pred, target) -> float:
    return math.sqrt(mse(pred, target))
