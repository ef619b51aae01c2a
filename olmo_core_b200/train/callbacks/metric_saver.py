"""Saves the most recent (and optionally selected-step) metrics as JSON files (metric_saver.py:18-85)."""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, List, Optional

from ...distributed.utils import get_rank
from .callback import Callback

__all__ = ["MetricSaverCallback"]


@dataclass
class MetricSaverCallback(Callback):
    enabled: bool = True
    metrics_to_capture: Optional[List[str]] = None
    fixed_steps: Optional[List[int]] = None
    fname: str = "metrics.json"

    def __post_init__(self):
        self._latest: Dict[str, float] = {}

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        if not self.enabled or get_rank() != 0:
            return
        keep = metrics if self.metrics_to_capture is None else {k: v for k, v in metrics.items() if k in self.metrics_to_capture}
        self._latest = dict(keep, step=step)
        if self.fixed_steps and step in self.fixed_steps:
            self.trainer.write_file(f"metrics_step{step}.json", json.dumps(self._latest))

    def post_train(self) -> None:
        if self.enabled and get_rank() == 0 and self._latest:
            self.trainer.write_file(self.fname, json.dumps(self._latest))
