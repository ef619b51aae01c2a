"""
Keeps the latest value of every (selected) metric on rank 0 and writes them as JSON files into the run's save folder:
at the end of the run, every ``save_interval`` steps and at ``fixed_steps``
(src/olmo_core/train/callbacks/metric_saver.py:14-85).
"""

from __future__ import annotations

import dataclasses
import json
import logging
from dataclasses import dataclass
from fnmatch import fnmatch
from typing import Any, Dict, List, Optional

from ...distributed.utils import get_rank
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["MetricSaverCallback"]


@dataclass
class MetricSaverCallback(Callback):
    step_metrics_fname: str = "metrics_step{step}.json"
    """File name of the per-step dumps; ``{step}`` is replaced by the step number."""
    final_metrics_fname: str = "metrics.json"
    metrics_to_capture: Optional[List[str]] = None
    """Glob patterns of the metrics to keep (``None``: all)."""
    save_interval: Optional[int] = None
    fixed_steps: Optional[List[int]] = None
    enabled: bool = True
    fname: Optional[str] = None
    """Older spelling of ``final_metrics_fname``."""

    _metrics: Optional[Dict[str, Any]] = dataclasses.field(default=None, repr=False)
    _metrics_step: int = dataclasses.field(default=0, repr=False)

    def __post_init__(self):
        if self.fname is not None:
            self.final_metrics_fname = self.fname

    @property
    def metrics(self) -> Optional[Dict[str, Any]]:
        """The latest value of every captured metric."""
        return self._metrics

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        if not self.enabled or get_rank() != 0:
            return
        if self._metrics is None:
            self._metrics = {}
        if step >= self._metrics_step:
            if self.metrics_to_capture is not None:
                metrics = {k: v for k, v in metrics.items() if any(fnmatch(k, pat) for pat in self.metrics_to_capture)}
            self._metrics.update(metrics)
            self._metrics["step"] = step
            self._metrics_step = step
        due = (self.save_interval is not None and step % self.save_interval == 0) or (
            self.fixed_steps is not None and step in self.fixed_steps)
        if due:
            dest = self.trainer.write_file(self.step_metrics_fname.format(step=step), json.dumps(self._metrics))
            log.info(f"Metrics for step {step} saved to '{dest}'")

    def _flush(self) -> None:
        if not self.enabled or get_rank() != 0:
            return
        if self._metrics is not None:
            dest = self.trainer.write_file(self.final_metrics_fname, json.dumps(self._metrics))
            log.info(f"Final metrics from step {self._metrics_step} saved to '{dest}'")
        self._metrics = None
        self._metrics_step = 0

    def post_train(self) -> None:
        self._flush()

    def close(self) -> None:
        self._flush()
