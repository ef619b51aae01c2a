"""Peak GPU memory per step (gpu_memory_monitor.py:16-80)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from ..common import ReduceType
from .callback import Callback

__all__ = ["GPUMemoryMonitorCallback"]


@dataclass
class GPUMemoryMonitorCallback(Callback):
    priority: ClassVar[int] = -1

    def __post_init__(self):
        self._capacity = 0

    def pre_train(self) -> None:
        if self.trainer.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats()
            self._capacity = torch.cuda.get_device_properties(self.trainer.device).total_memory

    def post_step(self) -> None:
        if self.trainer.device.type != "cuda":
            return
        gib = float(1 << 30)
        stats = torch.cuda.memory_stats()
        active = stats.get("active_bytes.all.peak", 0)
        reserved = stats.get("reserved_bytes.all.peak", 0)
        rec = self.trainer.record_metric
        rec("gpu_memory/peak active (GiB)", active / gib, reduce_type=ReduceType.max)
        rec("gpu_memory/peak reserved (GiB)", reserved / gib, reduce_type=ReduceType.max)
        if self._capacity:
            rec("gpu_memory/peak active (%)", 100 * active / self._capacity, reduce_type=ReduceType.max)
            rec("gpu_memory/peak reserved (%)", 100 * reserved / self._capacity, reduce_type=ReduceType.max)
        torch.cuda.reset_peak_memory_stats()
