"""Progress and metrics on the console (src/olmo_core/train/callbacks/console_logger.py:15-93)."""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from fnmatch import fnmatch
from typing import Dict, List, Optional

from ...utils import format_float, format_timedelta
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["ConsoleLoggerCallback"]


@dataclass
class ConsoleLoggerCallback(Callback):
    log_interval: int = 1
    metrics_log_interval: Optional[int] = None
    metrics: List[str] = field(default_factory=lambda: [
        "train/CE loss", "train/PPL", "train/Z loss", "train/load balancing loss", "train/router Z loss",
        "train/block */load imbalance", "gpu_memory/*", "optim/total grad norm", "optim/step skipped", "optim/LR*",
        "throughput/*", "checkpoint/*",
    ])

    def _wants_metrics(self, step: int) -> bool:
        every = self.metrics_log_interval or self.log_interval
        return step == 1 or (step > 1 and step % every == 0)

    def _marker(self, step: int, eta: bool = False) -> str:
        tr = self.trainer
        head = f"step={step}/{tr.max_steps or '???'},epoch={tr.epoch}"
        if eta and (remaining := tr.training_progress.time_remaining) is not None:
            text = format_timedelta(remaining).replace(", ", "")
            head += f",eta={text}{'(hard stop)' if tr.hard_stop else ''}"
        return f"[{head}]"

    def post_step(self) -> None:
        if not self._wants_metrics(self.step) and self.step % self.log_interval == 0:
            log.info(self._marker(self.step))

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        if not self._wants_metrics(step):
            return
        lines = [f"    {n}={format_float(v)}" for n, v in metrics.items() if any(fnmatch(n, p) for p in self.metrics)]
        log.info(self._marker(step, eta=True) + "\n" + "\n".join(lines))
