"""
Checkpoints at an explicit list of steps, e.g. the boundaries of a WSD-S learning-rate schedule
(src/olmo_core/train/callbacks/list_checkpointer.py:11-60).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import List, Optional, Set

from .checkpointer import CheckpointerCallback

log = logging.getLogger(__name__)

__all__ = ["ListCheckpointerCallback"]


@dataclass
class ListCheckpointerCallback(CheckpointerCallback):
    save_interval: int = 1_000_000_000  # effectively never: only ``save_steps`` trigger a save
    save_steps: Optional[List[int]] = None

    _save_steps_set: Set[int] = field(default_factory=set, init=False, repr=False)
    _last_saved_step: int = field(default=-1, init=False, repr=False)

    def __post_init__(self):
        super().__post_init__()
        if not self.save_steps:
            raise ValueError("'save_steps' must be provided (list of step indices to checkpoint).")
        self._save_steps_set = {int(s) for s in self.save_steps}

    def post_train_batch(self) -> None:
        if not self.enabled:
            return
        self._await_last_checkpoint(blocking=False)
        if not self.checkpoint_pending:
            self._flush_removals()
        step = int(self.step)
        if step in self._save_steps_set and step != self._last_saved_step:
            path = self._save()
            self._last_saved_step = step
            log.info(f"Saved checkpoint for listed step {step} -> {path}")
