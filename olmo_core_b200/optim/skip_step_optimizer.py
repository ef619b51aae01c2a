"""
Base class for optimizers that can skip an update when the loss or the gradient norm spikes
(src/olmo_core/optim/skip_step_optimizer.py:12-116). The decision is a 0/1 *tensor* multiplied into every
term of the update, so no host synchronisation happens on the training path.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.optim.optimizer import Optimizer

from ..utils import get_default_device

__all__ = ["SkipStepOptimizer"]


class SkipStepOptimizer(Optimizer):
    """
    Set :data:`latest_loss` and :data:`latest_grad_norm` before every :meth:`step`. The step proceeds iff
    both are within ``sigma_factor`` standard deviations above the mean of the previous values in a rolling
    window of ``rolling_interval_length``; until half a window has been seen every step proceeds.
    """

    def __init__(self, params, defaults: Dict[str, Any], rolling_interval_length: int = 128, sigma_factor: int = 6) -> None:
        super().__init__(params, defaults)
        self.rolling_interval_length = rolling_interval_length
        self.sigma_factor = sigma_factor
        self._losses: List[torch.Tensor] = []
        self._grad_norms: List[torch.Tensor] = []
        self._device: Optional[torch.device] = None

    @property
    def device(self) -> torch.device:
        if self._device is None:
            for group in self.param_groups:
                for p in group["params"]:
                    if p.numel() > 0:
                        self._device = p.device
                        return self._device
            self._device = get_default_device()
        return self._device

    def _push(self, history: List[torch.Tensor], value: torch.Tensor) -> None:
        history.append(value)
        del history[: max(0, len(history) - (self.rolling_interval_length + 1))]

    @property
    def latest_loss(self) -> Optional[torch.Tensor]:
        return self._losses[-1] if self._losses else None

    @latest_loss.setter
    def latest_loss(self, loss: torch.Tensor) -> None:
        self._push(self._losses, loss)

    @property
    def latest_grad_norm(self) -> Optional[torch.Tensor]:
        return self._grad_norms[-1] if self._grad_norms else None

    @latest_grad_norm.setter
    def latest_grad_norm(self, grad_norm: torch.Tensor) -> None:
        self._push(self._grad_norms, grad_norm)

    def get_step_factor(self) -> torch.Tensor:
        """1.0 to take the step, 0.0 to skip it (fp32 scalar tensor on the optimizer's device)."""
        if len(self._losses) < max(2, self.rolling_interval_length // 2):
            return torch.ones((), dtype=torch.float32, device=self.device)
        std, mean = torch.std_mean(torch.stack(self._losses[:-1]))
        ok = (self._losses[-1] - mean) <= self.sigma_factor * std
        if self._grad_norms:
            gstd, gmean = torch.std_mean(torch.stack(self._grad_norms[:-1]))
            ok = torch.logical_and(ok, (self._grad_norms[-1] - gmean) <= self.sigma_factor * gstd)
        return ok.float().to(self.device)

    @property
    def step_skipped(self) -> torch.Tensor:
        return 1 - self.get_step_factor()
