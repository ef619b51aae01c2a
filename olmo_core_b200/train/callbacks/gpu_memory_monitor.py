"""
Peak GPU memory per step under the metric names of the reference
(src/olmo_core/train/callbacks/gpu_memory_monitor.py:14-80), plus warnings when the allocator had to retry or ran out.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["GPUMemoryMonitorCallback"]

_GIB = float(1 << 30)


@dataclass
class GPUMemoryMonitorCallback(Callback):
    priority: ClassVar[int] = -1
    device_id: Optional[int] = None
    _num_alloc_retries: int = 0

    @property
    def device(self) -> torch.device:
        return torch.device("cuda") if self.device_id is None else torch.device(f"cuda:{self.device_id}")

    @property
    def device_name(self) -> str:
        return torch.cuda.get_device_name(self.device)

    @property
    def device_capacity(self) -> int:
        return torch.cuda.get_device_properties(self.device).total_memory

    def _active(self) -> bool:
        return torch.cuda.is_available() and self.trainer.device.type == "cuda"

    def pre_train(self) -> None:
        if not self._active():
            return
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.empty_cache()
        log.info(f"GPU capacity: {self.device_name} with {self.device_capacity / _GIB:.2f}GiB memory of which "
                 f"{torch.cuda.memory_allocated() / _GIB:.2f}GiB is currently allocated and "
                 f"{torch.cuda.memory_reserved() / _GIB:.2f}GiB is currently reserved.")

    def post_step(self) -> None:
        if not self._active():
            return
        stats = torch.cuda.memory_stats(self.device)
        capacity = self.device_capacity
        for label, key in (("active", "active_bytes.all.peak"), ("reserved", "reserved_bytes.all.peak")):
            peak = stats.get(key, 0)
            self.trainer.record_metric(f"gpu_memory/GPU {label} mem (GiB)", peak / _GIB)
            self.trainer.record_metric(f"gpu_memory/GPU {label} mem (%)", 100 * peak / capacity)
        retries = stats.get("num_alloc_retries", 0)
        if retries > self._num_alloc_retries:
            log.warning(f"{retries} CUDA memory allocation retries.")
            self._num_alloc_retries = retries
        if stats.get("num_ooms", 0) > 0:
            log.warning(f"{stats['num_ooms']} CUDA OOM errors thrown.")
        torch.cuda.reset_peak_memory_stats()
