"""Lion and its skip-step variant (API of src/olmo_core/optim/lion.py:12-172)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Type

import torch
from torch.optim.optimizer import Optimizer

from .config import OptimConfig
from .skip_step_optimizer import SkipStepOptimizer

__all__ = ["lion_step", "Lion", "SkipStepLion", "LionConfig", "SkipStepLionConfig"]


def lion_step(p: torch.Tensor, grad: Optional[torch.Tensor] = None, *, lr: float, weight_decay: float, exp_avg: torch.Tensor,
              betas: Tuple[float, float], step_factor: torch.Tensor) -> None:
    """
    Sign-momentum update: ``p <- p(1 - f lr wd) - lr sign(f (b1 m + (1-b1) g))``, ``m <- m(1 - f(1-b2)) + f(1-b2) g``.
    ``f`` is the 0/1 skip factor (sign(0) = 0 makes a skipped step a no-op).
    """
    g = grad if grad is not None else p.grad
    if g is None:
        return
    b1, b2 = betas
    p.mul_(1 - step_factor * (lr * weight_decay))
    update = (exp_avg * b1 + g * (1 - b1)) * step_factor
    p.add_(torch.sign(update), alpha=-lr)
    exp_avg.mul_(1 - step_factor * (1 - b2)).add_(step_factor * g, alpha=1 - b2)


class Lion(Optimizer):
    def __init__(self, params, lr: float = 1e-4, betas: Tuple[float, float] = (0.9, 0.99), weight_decay: float = 0.0):
        assert lr > 0.0 and all(0.0 <= b <= 1.0 for b in betas)
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None) -> None:
        if closure is not None:
            with torch.enable_grad():
                closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    state["exp_avg"] = torch.zeros_like(p)
                    state["step_factor"] = torch.tensor(1.0, device=p.device)
                lion_step(p, lr=group["lr"], weight_decay=group["weight_decay"], betas=group["betas"],
                          exp_avg=state["exp_avg"], step_factor=state["step_factor"])


class SkipStepLion(SkipStepOptimizer):
    def __init__(self, params, lr: float = 1e-4, betas: Tuple[float, float] = (0.9, 0.99), weight_decay: float = 0.0,
                 rolling_interval_length: int = 128, sigma_factor: int = 6) -> None:
        assert lr > 0.0 and all(0.0 <= b <= 1.0 for b in betas)
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay),
                         rolling_interval_length=rolling_interval_length, sigma_factor=sigma_factor)
        self._step_skipped: Optional[torch.Tensor] = None

    @property
    def step_skipped(self) -> torch.Tensor:
        return self._step_skipped if self._step_skipped is not None else torch.tensor(0.0)

    @torch.no_grad()
    def step(self, closure=None) -> None:
        if closure is not None:
            with torch.enable_grad():
                closure()
        f = self.get_step_factor()
        self._step_skipped = 1 - f
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    state["exp_avg"] = torch.zeros_like(p)
                lion_step(p, lr=group["lr"], weight_decay=group["weight_decay"], betas=group["betas"],
                          exp_avg=state["exp_avg"], step_factor=f)


@OptimConfig.register("lion")
@dataclass
class LionConfig(OptimConfig[Lion]):
    lr: float = 1e-4
    betas: Tuple[float, float] = (0.9, 0.99)
    weight_decay: float = 0.0

    @classmethod
    def optimizer(cls) -> Type[Lion]:
        return Lion


@OptimConfig.register("skip_step_lion")
@dataclass
class SkipStepLionConfig(OptimConfig[SkipStepLion]):
    lr: float = 1e-4
    betas: Tuple[float, float] = (0.9, 0.99)
    weight_decay: float = 0.0
    rolling_interval_length: int = 128
    sigma_factor: int = 6

    @classmethod
    def optimizer(cls) -> Type[SkipStepLion]:
        return SkipStepLion
