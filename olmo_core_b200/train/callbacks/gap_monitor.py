"""
GAP monitor: max / mean / variance of Gradients, Activations (and their gradients) and Parameters, per module
and parameter (metric names of src/olmo_core/train/callbacks/gap_monitor.py:26-342), plus optional dumps of
gradient tensors to the save folder for offline analysis.

Activations are observed with forward hooks and their gradients with backward pre-hooks on every sub-module;
statistics are computed on the device and recorded as tensors, so the monitor adds no host synchronisation.
Weight gradients are read from the fused ``main_grad`` buffers where a parameter has one.
"""

from __future__ import annotations

import dataclasses
import functools
import logging
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ...distributed.utils import get_local_tensor, get_rank
from ...io import join_path
from ..common import MetricMergeStrategy, ReduceType
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["GAPMonitorCallback"]


@dataclass
class GAPMonitorCallback(Callback):
    enabled: bool = True
    monitor: Optional[bool] = None
    """Record statistics (default: on when the callback is enabled)."""
    interval: int = 1
    dump_gradients: Optional[bool] = None
    dump_gradients_start_step: int = 0
    dump_gradients_end_step: Optional[int] = None
    dump_gradients_step_interval: int = 1
    dump_gradients_save_first_n: Optional[int] = None
    """Keep only the first N rows (dim 0) of every dumped gradient."""

    _handles: Optional[list] = dataclasses.field(default=None, repr=False)
    _local_batch_size_instances: int = dataclasses.field(default=1, repr=False)
    _dry_run_complete: bool = dataclasses.field(default=False, repr=False)

    def __post_init__(self):
        if not self.enabled:
            if self.monitor or self.dump_gradients:
                raise ValueError("Cannot set monitor or dump_gradients to True when enabled=False.")
            return
        self.monitor = True if self.monitor is None else self.monitor
        self.dump_gradients = False if self.dump_gradients is None else self.dump_gradients
        if not self.monitor and not self.dump_gradients:
            raise ValueError("enabled=True but both monitor and dump_gradients are False.")
        if self.dump_gradients:
            if self.dump_gradients_start_step < 0:
                raise ValueError(f"dump_gradients_start_step must be non-negative, got {self.dump_gradients_start_step}")
            if self.dump_gradients_step_interval <= 0:
                raise ValueError(f"dump_gradients_step_interval must be positive, got {self.dump_gradients_step_interval}")
            if self.dump_gradients_save_first_n is not None and self.dump_gradients_save_first_n <= 0:
                raise ValueError(f"dump_gradients_save_first_n must be positive, got {self.dump_gradients_save_first_n}")

    def _model(self) -> nn.Module:
        return self.trainer.train_module.model

    def post_attach(self) -> None:
        if self.enabled and not hasattr(self.trainer.train_module, "model"):
            raise ValueError(f"{type(self).__name__} needs a train module with a 'model'.")

    def pre_train(self) -> None:
        if not self.enabled or not self.monitor:
            return
        self._reset()
        self._handles = []
        for name, module in self._model().named_modules():
            if name == "":
                continue
            self._handles.append(module.register_forward_hook(functools.partial(self.forward_hook, module_name=name)))
            self._handles.append(module.register_full_backward_pre_hook(functools.partial(self.backward_hook, module_name=name)))

    def pre_step(self, batch: Dict[str, Any]) -> None:
        if self.enabled and self.monitor:
            self._dry_run_complete = True  # hooks also fire during the trainer's dry run, when nothing may be recorded
            self._local_batch_size_instances = batch["input_ids"].shape[0]

    @staticmethod
    def _grad_of(p: torch.Tensor) -> Optional[torch.Tensor]:
        g = getattr(p, "main_grad", None)
        return g if g is not None else p.grad

    def pre_optim_step(self) -> None:
        if not self.enabled:
            return
        if self.monitor:
            for name, p in self._model().named_parameters():
                self.record_tensor_stats(name, p, "param")
                g = self._grad_of(p)
                if g is not None:
                    self.record_tensor_stats(name, g, "grad")
        if self.dump_gradients:
            self._dump_gradients()

    def forward_hook(self, module: nn.Module, args, output, module_name: str) -> None:
        del module, args
        if isinstance(output, tuple):
            output = output[0]
        if isinstance(output, torch.Tensor):
            self.record_tensor_stats(module_name, output, "activation")

    def backward_hook(self, module: nn.Module, grad_output, module_name: str) -> None:
        del module
        if isinstance(grad_output, tuple):
            grad_output = grad_output[0]
        if isinstance(grad_output, torch.Tensor):
            self.record_tensor_stats(module_name, grad_output, "activation_grad")

    @torch.no_grad()
    def record_tensor_stats(self, name: str, tensor: torch.Tensor, kind: str) -> None:
        if not self.enabled or not self.monitor or not self._dry_run_complete:
            return
        if self.step % self.interval != 0 or tensor.numel() <= 1:
            return
        rec = self.trainer.record_metric
        prefix = f"gap/{kind}s/{name}"
        t = get_local_tensor(tensor.detach())
        if kind in ("activation", "activation_grad"):
            if t.ndim <= 1:
                return
            rows = t.reshape(t.shape[0], -1).float()
            var, mean = torch.var_mean(rows, dim=-1)
            # micro-batches of a step are merged: max of maxima, per-instance averages summed over micro-batches
            rec(f"{prefix}/max", rows.abs().max(), reduce_type=ReduceType.max, merge_strategy=MetricMergeStrategy.max)
            rec(f"{prefix}/mean", mean.sum() / self._local_batch_size_instances, reduce_type=ReduceType.mean,
                merge_strategy=MetricMergeStrategy.sum)
            rec(f"{prefix}/var", var.sum() / self._local_batch_size_instances, reduce_type=ReduceType.mean,
                merge_strategy=MetricMergeStrategy.sum)
        else:
            flat = t.float()
            var, mean = torch.var_mean(flat)
            sharded = getattr(getattr(tensor, "_shard_info", None), "sharded", False)
            rec(f"{prefix}/max", flat.abs().max(), reduce_type=ReduceType.max)
            rec(f"{prefix}/mean", mean, reduce_type=ReduceType.mean if sharded else None)
            rec(f"{prefix}/var", var, reduce_type=ReduceType.mean if sharded else None)

    def _dump_gradients(self) -> None:
        step = self.step
        if step < self.dump_gradients_start_step:
            return
        if self.dump_gradients_end_step is not None and step > self.dump_gradients_end_step:
            return
        if (step - self.dump_gradients_start_step) % self.dump_gradients_step_interval != 0:
            return
        out: Dict[str, torch.Tensor] = {}
        for name, p in self._model().named_parameters():
            g = self._grad_of(p)
            if g is None:
                continue
            g = get_local_tensor(g.detach())
            if self.dump_gradients_save_first_n is not None and g.ndim >= 1:
                g = g[: self.dump_gradients_save_first_n]
            out[name] = g.to("cpu", copy=True)
        folder = self.trainer.work_dir / "gradient_dumps" / f"step{step}"
        folder.mkdir(parents=True, exist_ok=True)
        path = folder / f"rank{get_rank()}.pt"
        torch.save(out, path)
        self.trainer.run_bookkeeping_op(self.trainer.persist_working_file, path, op_name=f"persist {path}", distributed=False)
        log.info(f"Dumped {len(out)} gradients for step {step} to '{join_path(self.trainer.save_folder, 'gradient_dumps')}'")

    def close(self) -> None:
        self._reset()

    def _reset(self) -> None:
        for h in self._handles or []:
            h.remove()
        self._handles = None


def var_mean(tensor: torch.Tensor, dim: Optional[int] = None):
    """``torch.var_mean`` that also takes a sharded ``DTensor`` (reduced to full values; unbiased variance)."""
    import math

    from torch.distributed.tensor import DTensor

    from ...distributed.utils import get_full_tensor

    if not isinstance(tensor, DTensor):
        return torch.var_mean(tensor, dim=dim)
    numel = tensor.numel() if dim is None else tensor.size(dim)
    mean = get_full_tensor(tensor.mean(dim=dim))
    spread = get_full_tensor(torch.linalg.vector_norm(tensor - mean, dim=dim)) / math.sqrt(max(1, numel - 1))
    return spread ** 2, mean
