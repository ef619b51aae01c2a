"""Streaming metrics for in-loop evaluation (src/olmo_core/eval/metrics.py:13-93)."""

from __future__ import annotations

from abc import ABCMeta, abstractmethod
from typing import Optional, Union

import torch
import torch.distributed as dist

from ..distributed.utils import is_distributed
from ..utils import get_default_device

__all__ = ["Metric", "MeanMetric"]


class Metric(metaclass=ABCMeta):
    def __init__(self, device: Optional[torch.device] = None, process_group: Optional[dist.ProcessGroup] = None):
        self.device = device if device is not None else get_default_device()
        self.process_group = process_group

    @abstractmethod
    def update(self, *args, **kwargs) -> None:
        raise NotImplementedError

    @abstractmethod
    def compute(self) -> torch.Tensor:
        """The metric over everything seen so far on all ranks."""
        raise NotImplementedError

    @abstractmethod
    def reset(self) -> None:
        raise NotImplementedError

    def as_tensor(self, value: Union[float, torch.Tensor]) -> torch.Tensor:
        if not isinstance(value, torch.Tensor):
            value = torch.tensor(value)
        return value.to(device=self.device, non_blocking=self.device.type != "cpu")


class MeanMetric(Metric):
    """Weighted mean of a stream of values; numerator and denominator travel in ONE all-reduce."""

    def __init__(self, device: Optional[torch.device] = None, process_group: Optional[dist.ProcessGroup] = None):
        super().__init__(device=device, process_group=process_group)
        self._acc = torch.zeros(2, dtype=torch.float32, device=self.device)  # [weighted sum, weight]

    @property
    def weighted_sum(self) -> torch.Tensor:
        return self._acc[0]

    @property
    def weight(self) -> torch.Tensor:
        return self._acc[1]

    def update(self, value: Union[float, torch.Tensor], weight: Union[float, torch.Tensor] = 1.0) -> None:
        value = self.as_tensor(value).float()
        if value.numel() == 0:
            return
        weight = torch.broadcast_to(self.as_tensor(weight).float(), value.shape)
        self._acc[0] += (value * weight).sum()
        self._acc[1] += weight.sum()

    def compute(self) -> torch.Tensor:
        acc = self._acc.clone()
        if is_distributed():
            dist.all_reduce(acc, group=self.process_group)
        return acc[0] / acc[1]

    def reset(self) -> None:
        self._acc.zero_()
