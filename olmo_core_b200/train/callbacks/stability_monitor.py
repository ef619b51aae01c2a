"""
Loss / gradient-norm spike detection (metrics of src/olmo_core/train/callbacks/stability_monitor.py:15-135).

A value is a *spike* when it exceeds ``mean + threshold_std * std`` of the previous ``window_size`` values.
``spike/SpikeScore`` is the fraction of spiking steps over the last ``rolling_window`` steps (reported once that
window is full), ``spike/SpikeScore (total)`` the fraction over the whole run.
"""

from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict

from ..common import OPTIM_GRAD_NORM_METRIC, TRAIN_CE_LOSS_METRIC
from .callback import Callback

__all__ = ["StabilityMonitorCallback"]


@dataclass
class StabilityMonitorCallback(Callback):
    window_size: int = 128
    rolling_window: int = 10000
    threshold_std: float = 6.0
    enabled: bool = True
    loss_metric_name: str = TRAIN_CE_LOSS_METRIC
    grad_norm_metric_name: str = OPTIM_GRAD_NORM_METRIC

    _loss_history: Deque[float] = field(default_factory=deque, repr=False)
    _grad_norm_history: Deque[float] = field(default_factory=deque, repr=False)
    _spike_history: Deque[bool] = field(default_factory=deque, repr=False)
    _total_spike_count: int = 0
    _total_step_count: int = 0

    def state_dict(self) -> Dict[str, Any]:
        return {
            "loss_history": list(self._loss_history),
            "grad_norm_history": list(self._grad_norm_history),
            "spike_history": list(self._spike_history),
            "total_spike_count": self._total_spike_count,
            "total_step_count": self._total_step_count,
        }

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._loss_history = deque(state_dict.get("loss_history", []))
        self._grad_norm_history = deque(state_dict.get("grad_norm_history", []))
        self._spike_history = deque(state_dict.get("spike_history", []))
        self._total_spike_count = state_dict.get("total_spike_count", 0)
        self._total_step_count = state_dict.get("total_step_count", 0)

    def _is_spike(self, value: float, history) -> bool:
        n = len(history)
        if n < self.window_size:
            return False
        mean = sum(history) / n
        std = math.sqrt(sum((x - mean) ** 2 for x in history) / n)
        return std >= 1e-10 and value > mean + self.threshold_std * std

    def _observe(self, value: float, history: Deque[float]) -> bool:
        spike = self._is_spike(value, history)
        history.append(value)
        while len(history) > self.window_size:
            history.popleft()
        return spike

    def pre_log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        del step
        if not self.enabled:
            return
        spike = False
        if self.loss_metric_name in metrics:
            spike |= self._observe(metrics[self.loss_metric_name], self._loss_history)
        if self.grad_norm_metric_name in metrics:
            spike |= self._observe(metrics[self.grad_norm_metric_name], self._grad_norm_history)
        self._spike_history.append(spike)
        while len(self._spike_history) > self.rolling_window:
            self._spike_history.popleft()
        self._total_step_count += 1
        self._total_spike_count += int(spike)
        if len(self._spike_history) >= self.rolling_window:
            metrics["spike/SpikeScore"] = sum(self._spike_history) / self.rolling_window
        if self._total_step_count >= self.window_size:
            metrics["spike/SpikeScore (total)"] = self._total_spike_count / self._total_step_count
