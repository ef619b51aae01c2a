"""Manual garbage collection at fixed steps so that all ranks pause together (garbage_collector.py:13-53)."""

from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import ClassVar, Optional

from .callback import Callback

__all__ = ["GarbageCollectorCallback"]


@dataclass
class GarbageCollectorCallback(Callback):
    gc_interval: int = 1000
    enabled: bool = True
    priority: ClassVar[int] = -1

    def __post_init__(self):
        self._was_enabled: Optional[bool] = None

    def pre_train(self) -> None:
        if not self.enabled:
            return
        self._was_enabled = gc.isenabled()
        gc.disable()
        gc.collect(1)

    def post_step(self) -> None:
        if self.enabled and self.step % self.gc_interval == 0:
            gc.collect(1)

    def close(self) -> None:
        if self.enabled and self._was_enabled:
            gc.enable()
        self._was_enabled = None

    post_train = close

    def on_error(self, exc: BaseException) -> None:
        self.close()
