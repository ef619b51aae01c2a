"""
Throughput monitor: tokens/s, batches/s, FLOP/s and MFU per device
(metric names and definitions of src/olmo_core/train/callbacks/speed_monitor.py:18-215).

``MFU = 100 * num_flops_per_token(seq_len) * tokens / dt / peak``; the first step is excluded. Wall-clock
numbers use ``perf_counter`` like the reference; in addition the step is timed on the device with CUDA
events (``throughput/device/step time (device ms)``), which does not include host-side stalls.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Optional

import torch

from ...config import DType
from ...distributed.utils import get_world_size
from ..common import ReduceType
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["SpeedMonitorCallback", "peak_flops_per_second"]

# Dense (no 2:4 sparsity) bf16/fp16 tensor-core peaks used as the MFU denominator.
_PEAKS = (("B200", 2.25e15), ("H100 NVL", 0.8355e15), ("H100 PCIe", 0.7565e15), ("H100", 0.9895e15), ("H200", 0.9895e15))
_DEFAULT_PEAK = 0.312e15  # A100 and unknown devices


def peak_flops_per_second(device_name: str) -> int:
    for key, peak in _PEAKS:
        if all(part in device_name for part in key.split()):
            return int(peak)
    return int(_DEFAULT_PEAK)


@dataclass
class SpeedMonitorCallback(Callback):
    priority: ClassVar[int] = -2

    num_flops_per_token: Optional[int] = None
    num_params: Optional[int] = None
    device_peak_flops_per_second: Optional[int] = None

    def __post_init__(self):
        self.reset()
        self._total_steps = self._total_tokens = self._total_flops = 0
        self._start_time = self._last_logged = self._load_start = self._load_time = 0.0
        self._step_tokens = self._step_seq_len = self._step_flops = 0
        self._parallel_degree = 1
        self._tps_avg: Optional[float] = None
        self._mfu_avg: Optional[float] = None
        self._ev_start = self._ev_end = None

    def reset(self) -> None:
        self._first_step = True
        self._bps_avg: Optional[float] = None

    @property
    def bps_avg(self) -> Optional[float]:
        return self._bps_avg

    @property
    def tps_avg(self) -> Optional[float]:
        return self._tps_avg

    @property
    def mfu_avg(self) -> Optional[float]:
        return self._mfu_avg

    def _flops_per_token(self, seq_len: int) -> Optional[int]:
        if self.num_flops_per_token is not None:
            return self.num_flops_per_token
        return self.trainer.train_module.num_flops_per_token(seq_len)

    def pre_train(self) -> None:
        self._first_step = True
        tm = self.trainer.train_module
        if self.trainer.dp_process_group is not None:
            self._parallel_degree = get_world_size() // get_world_size(self.trainer.dp_process_group)
        model = getattr(tm, "model", None)
        if self.num_params is None and model is not None and hasattr(model, "num_non_embedding_params"):
            self.num_params = model.num_non_embedding_params
        if self.device_peak_flops_per_second is None and self.trainer.device.type == "cuda":
            dp = getattr(tm, "dp_config", None)
            half = getattr(tm, "autocast_precision", None) == torch.bfloat16 or (dp is not None and dp.param_dtype == DType.bfloat16)
            if half:
                name = torch.cuda.get_device_name(self.trainer.device)
                self.device_peak_flops_per_second = peak_flops_per_second(name)
                log.info(f"Device: {name}, Device peak Flops/s: {self.device_peak_flops_per_second}")

    def pre_load_batch(self) -> None:
        self._load_start = time.perf_counter()

    def pre_step(self, batch: Dict[str, Any]) -> None:
        self._load_time = time.perf_counter() - self._load_start
        if self.trainer.device.type == "cuda":
            self._ev_start = torch.cuda.Event(enable_timing=True)
            self._ev_end = torch.cuda.Event(enable_timing=True)
            self._ev_start.record()
        if self._first_step:
            return
        self._total_steps += 1
        if "input_ids" in batch:
            self._step_tokens = batch["input_ids"].numel() // self._parallel_degree
            self._step_seq_len = batch["input_ids"].shape[1]
            self._total_tokens += self._step_tokens
            per_tok = self._flops_per_token(self._step_seq_len)
            self._step_flops = per_tok * self._step_tokens if per_tok is not None else 0
            self._total_flops += self._step_flops

    def post_step(self) -> None:
        now = time.perf_counter()
        rec = self.trainer.record_metric
        rec("throughput/device/data loading (s)", self._load_time, reduce_type=ReduceType.max)
        if self._ev_end is not None:
            self._ev_end.record()
        if self._first_step:
            self._total_steps = self._total_tokens = self._total_flops = 0
            self._start_time = self._last_logged = now
            self._first_step = False
            return
        dt, total = now - self._last_logged, now - self._start_time
        self._last_logged = now
        if self._step_tokens and self._total_tokens:
            self._tps_avg = self._total_tokens / total
            rec("throughput/device/TPS", self._step_tokens / dt)
            rec("throughput/device/TPS (actual avg)", self._tps_avg)
        rec("throughput/total tokens", self.trainer.global_train_tokens_seen)
        if self.num_params:
            rec("throughput/chinchilla multiple", self.trainer.global_train_tokens_seen / (20 * self.num_params))
        flops_ps = flops_avg = None
        if self._step_flops and self._total_flops:
            flops_ps, flops_avg = self._step_flops / dt, self._total_flops / total
            rec("throughput/device/flopsPS", flops_ps)
            rec("throughput/device/flopsPS (actual avg)", flops_avg)
            rec("throughput/total petaflops", self.trainer.global_train_petaflops)
        self._bps_avg = self._total_steps / total
        rec("throughput/device/BPS", 1 / dt)
        rec("throughput/device/BPS (actual avg)", self._bps_avg)
        rec("throughput/device/data loading (%)", 100 * self._load_time / dt, reduce_type=ReduceType.max)
        if self.device_peak_flops_per_second and flops_ps is not None and flops_avg is not None:
            self._mfu_avg = 100 * flops_avg / self.device_peak_flops_per_second
            rec("throughput/device/MFU", 100 * flops_ps / self.device_peak_flops_per_second)
            rec("throughput/device/MFU (actual avg)", self._mfu_avg)

    def pre_log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        # By the time metrics are flushed the step's events have completed, so reading them does not stall.
        if self._ev_start is not None and self._ev_end is not None and self._ev_end.query():
            metrics["throughput/device/step time (device ms)"] = self._ev_start.elapsed_time(self._ev_end)
