"""Learning-rate schedulers with the reference's exact arithmetic (include/nn/schedulers.hpp:86-781).

Every ``step()`` increments the step counter first. Quirks that are kept on purpose because
configs written for the reference depend on them:

* ``step_lr`` multiplies the *current* LR (not the base LR) every ``step_size`` steps.
* ``linear_warmup`` / ``warmup_cosine_annealing`` start at ``start + (base-start)/warmup`` and use
  ``(step+1)/warmup`` as progress.
* ``warmup_cosine_annealing`` computes ``total_steps - warmup_steps`` in unsigned 64-bit
  arithmetic. The factory reads ``total_steps`` (default 1000) and ignores ``T_max``/``base_lr``
  (``:744-750``), so the stock GPT-2 / ResNet configs (warmup 2000, no total_steps) wrap around to
  ~1.8e19 decay steps and the LR simply stays at the base LR after warm-up.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np

_F = np.float32
_PI = _F(math.pi)


class Scheduler:
    TYPE = "no_op"

    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.base_lr = float(_F(optimizer.get_learning_rate())) if optimizer is not None else 0.0
        self.current_step = 0

    def get_lr(self) -> float:
        return self.optimizer.get_learning_rate() if self.optimizer is not None else self.base_lr

    def set_lr(self, lr) -> None:
        if self.optimizer is not None:
            self.optimizer.set_learning_rate(float(_F(lr)))

    def step(self, metric: Optional[float] = None) -> None:
        self.current_step += 1

    def reset(self) -> None:
        self.current_step = 0
        self.set_lr(self.base_lr)

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, d: dict) -> None:
        self.__dict__.update(d)


class NoOp(Scheduler):
    TYPE = "no_op"


class StepLR(Scheduler):
    TYPE = "step_lr"

    def __init__(self, optimizer, step_size: int = 10, gamma: float = 0.1):
        super().__init__(optimizer)
        self.step_size, self.gamma = int(step_size), _F(gamma)

    def step(self, metric=None):
        self.current_step += 1
        if self.current_step % self.step_size == 0:
            self.set_lr(_F(self.get_lr()) * self.gamma)


class MultiStepLR(Scheduler):
    TYPE = "multi_step_lr"

    def __init__(self, optimizer, milestones: List[int] = (), gamma: float = 0.1):
        super().__init__(optimizer)
        self.milestones, self.gamma, self.idx = sorted(int(m) for m in milestones), _F(gamma), 0

    def step(self, metric=None):
        self.current_step += 1
        if self.idx < len(self.milestones) and self.current_step >= self.milestones[self.idx]:
            self.set_lr(_F(self.get_lr()) * self.gamma)
            self.idx += 1

    def reset(self):
        super().reset()
        self.idx = 0


class ExponentialLR(Scheduler):
    TYPE = "exponential_lr"

    def __init__(self, optimizer, gamma: float = 0.95):
        super().__init__(optimizer)
        self.gamma = _F(gamma)

    def step(self, metric=None):
        self.current_step += 1
        self.set_lr(_F(self.get_lr()) * self.gamma)


def _cos_blend(base, eta_min, x):
    base, eta_min = _F(base), _F(eta_min)
    return eta_min + (base - eta_min) * (_F(1.0) + _F(math.cos(float(x)))) / _F(2.0)


class CosineAnnealingLR(Scheduler):
    TYPE = "cosine_annealing_lr"

    def __init__(self, optimizer, T_max: int = 100, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.T_max, self.eta_min = int(T_max), float(eta_min)

    def step(self, metric=None):
        self.current_step += 1
        s = self.current_step % self.T_max
        self.set_lr(_cos_blend(self.base_lr, self.eta_min, _PI * _F(s) / _F(self.T_max)))


class CosineAnnealingWarmRestarts(Scheduler):
    TYPE = "cosine_annealing_warm_restarts"

    def __init__(self, optimizer, T_0: int = 10, T_mult: int = 1, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.T_0, self.T_mult, self.eta_min = int(T_0), int(T_mult), float(eta_min)
        self.T_cur, self.T_i = 0, int(T_0)

    def step(self, metric=None):
        self.current_step += 1
        self.T_cur += 1
        if self.T_cur >= self.T_i:
            self.T_cur = 0
            self.T_i *= self.T_mult
        self.set_lr(_cos_blend(self.base_lr, self.eta_min, _PI * _F(self.T_cur) / _F(self.T_i)))

    def reset(self):
        super().reset()
        self.T_cur, self.T_i = 0, self.T_0


class LinearWarmup(Scheduler):
    TYPE = "linear_warmup"

    def __init__(self, optimizer, warmup_steps: int = 100, start_lr: float = 0.0):
        super().__init__(optimizer)
        self.warmup_steps, self.start_lr = int(warmup_steps), float(start_lr)
        if self.warmup_steps > 0:
            self.set_lr(_F(self.start_lr) + (_F(self.base_lr) - _F(self.start_lr)) / _F(self.warmup_steps))

    def _warm(self):
        progress = _F(self.current_step + 1) / _F(self.warmup_steps)
        self.set_lr(_F(self.start_lr) + progress * (_F(self.base_lr) - _F(self.start_lr)))

    def step(self, metric=None):
        self.current_step += 1
        if self.current_step < self.warmup_steps:
            self._warm()
        elif self.warmup_steps == 0 or self.current_step == self.warmup_steps - 1:
            self.set_lr(self.base_lr)

    def is_warmup_complete(self) -> bool:
        return self.warmup_steps == 0 or self.current_step >= self.warmup_steps - 1


class WarmupCosineAnnealing(LinearWarmup):
    TYPE = "warmup_cosine_annealing"

    def __init__(self, optimizer, warmup_steps: int = 100, total_steps: int = 1000, start_lr: float = 0.0,
                 eta_min: float = 0.0):
        super().__init__(optimizer, warmup_steps, start_lr)
        self.total_steps, self.eta_min = int(total_steps), float(eta_min)

    def step(self, metric=None):
        self.current_step += 1
        if self.current_step < self.warmup_steps:
            self._warm()
            return
        decay = (self.total_steps - self.warmup_steps) & 0xFFFFFFFFFFFFFFFF  # size_t arithmetic
        cur = self.current_step - self.warmup_steps
        progress = _F(cur) / _F(decay) if decay else _F(np.inf if cur else np.nan)
        progress = min(progress, _F(1.0)) if not np.isnan(progress) else _F(1.0)
        self.set_lr(_cos_blend(self.base_lr, self.eta_min, _PI * progress))


class ReduceLROnPlateau(Scheduler):
    TYPE = "reduce_lr_on_plateau"

    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4,
                 min_lr: float = 0.0):
        super().__init__(optimizer)
        self.mode, self.factor, self.patience = mode, float(factor), int(patience)
        self.threshold, self.min_lr = float(threshold), float(min_lr)
        self.best = 1e10 if mode != "max" else -1e10
        self.bad = 0

    def step(self, metric=None):
        self.current_step += 1
        if metric is None:
            return
        better = metric > self.best + self.threshold if self.mode == "max" else metric < self.best - self.threshold
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                self.set_lr(max(self.get_lr() * self.factor, self.min_lr))
                self.bad = 0

    def reset(self):
        super().reset()
        self.best, self.bad = (1e10 if self.mode != "max" else -1e10), 0


class PolynomialLR(Scheduler):
    TYPE = "polynomial_lr"

    def __init__(self, optimizer, total_steps: int = 100, power: float = 1.0, end_lr: float = 0.0):
        super().__init__(optimizer)
        self.total_steps, self.power, self.end_lr = int(total_steps), float(power), float(end_lr)

    def step(self, metric=None):
        self.current_step += 1
        progress = min(_F(self.current_step) / _F(self.total_steps), _F(1.0))
        self.set_lr((_F(self.base_lr) - _F(self.end_lr)) * _F(float(_F(1.0) - progress) ** self.power) + _F(self.end_lr))


class OneCycleLR(Scheduler):
    TYPE = "one_cycle_lr"

    def __init__(self, optimizer, max_lr: float = 0.1, total_steps: int = 100, pct_start: float = 0.3,
                 div_factor: float = 25.0, final_div_factor: float = 1e4):
        super().__init__(optimizer)
        self.max_lr, self.total_steps = float(max_lr), int(total_steps)
        self.initial_lr = float(_F(max_lr) / _F(div_factor))
        self.min_lr = float(_F(self.initial_lr) / _F(final_div_factor))
        self.step_up = int(_F(self.total_steps) * _F(pct_start))
        self.step_down = self.total_steps - self.step_up
        self.set_lr(self.initial_lr)

    def step(self, metric=None):
        self.current_step += 1
        if self.current_step <= self.step_up:
            progress = _F(self.current_step) / _F(self.step_up)
            lr = _F(self.initial_lr) + progress * (_F(self.max_lr) - _F(self.initial_lr))
        else:
            progress = _F(self.current_step - self.step_up) / _F(self.step_down)
            lr = _cos_blend(self.max_lr, self.min_lr, _PI * progress)
        self.set_lr(lr)


SCHEDULERS: Dict[str, type] = {c.TYPE: c for c in (NoOp, StepLR, MultiStepLR, ExponentialLR, CosineAnnealingLR,
                                                   CosineAnnealingWarmRestarts, LinearWarmup, WarmupCosineAnnealing,
                                                   ReduceLROnPlateau, PolynomialLR, OneCycleLR)}

_KEYS = {
    "step_lr": ("step_size", "gamma"), "multi_step_lr": ("milestones", "gamma"), "exponential_lr": ("gamma",),
    "cosine_annealing_lr": ("T_max", "eta_min"), "cosine_annealing_warm_restarts": ("T_0", "T_mult", "eta_min"),
    "linear_warmup": ("warmup_steps", "start_lr"),
    "warmup_cosine_annealing": ("warmup_steps", "total_steps", "start_lr", "eta_min"),
    "reduce_lr_on_plateau": ("mode", "factor", "patience", "threshold", "min_lr"),
    "polynomial_lr": ("total_steps", "power", "end_lr"),
    "one_cycle_lr": ("max_lr", "total_steps", "pct_start", "div_factor", "final_div_factor"), "no_op": (),
}


def create_scheduler(cfg: Optional[dict], optimizer) -> Scheduler:
    """Factory from a config block ``{"type": ..., ...}``; keys the reference factory does not read
    (``base_lr``, ``T_max`` on the warm-up schedulers ...) are ignored, unknown types give ``no_op``."""
    cfg = dict(cfg or {})
    t = cfg.get("type", "no_op")
    if t not in SCHEDULERS:
        return NoOp(optimizer)
    kw = {k: cfg[k] for k in _KEYS[t] if k in cfg}
    return SCHEDULERS[t](optimizer, **kw)
