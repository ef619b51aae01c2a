"""Optimizer that updates nothing but keeps the skip-step statistics (src/olmo_core/optim/noop.py:10-94)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Type

import torch

from .config import OptimConfig
from .skip_step_optimizer import SkipStepOptimizer

__all__ = ["NoOpOptimizer", "NoOpConfig"]


class NoOpOptimizer(SkipStepOptimizer):
    """For eval-only or statistics-gathering runs: parameters never change, step counters advance."""

    def __init__(self, params, lr: float = 1e-3, rolling_interval_length: int = 128, sigma_factor: int = 6) -> None:
        super().__init__(params, dict(lr=lr), rolling_interval_length=rolling_interval_length, sigma_factor=sigma_factor)
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
                    state["step"] = torch.zeros((), dtype=torch.float32, device=p.device)
                state["step"] += f


@OptimConfig.register("noop")
@dataclass
class NoOpConfig(OptimConfig[NoOpOptimizer]):
    lr: float = 1e-3
    rolling_interval_length: int = 128
    sigma_factor: int = 6

    @classmethod
    def optimizer(cls) -> Type[NoOpOptimizer]:
        return NoOpOptimizer
