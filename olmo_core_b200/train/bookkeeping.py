"""
Host-side bookkeeping of the trainer: metric recording, windowed cross-rank metric reduction off the critical
path, cancellation that all ranks agree on, and thread pools for background work
(behaviour of src/olmo_core/train/trainer.py:1037-1126 and :1252-1442).

Collectives issued for bookkeeping run on a dedicated CPU (gloo) process group from ONE worker thread, in
submission order, so they can never interleave with the NCCL stream of the training step; with
``async_bookkeeping`` off the same operations run inline.
"""

from __future__ import annotations

import logging
import math
import time
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Callable, Dict, Optional, TypeVar, Union

import torch
import torch.distributed as dist

from ..distributed.utils import (
    all_reduce_value,
    backend_supports_cpu,
    broadcast_object,
    get_global_rank,
    get_local_tensor,
    get_rank,
    is_distributed,
)
from ..utils import cuda_sync_debug_mode, get_default_thread_count
from .common import TRAIN_CE_LOSS_METRIC, TRAIN_PPL_METRIC, MetricMergeStrategy, ReduceType
from .utils import check_metrics_consistent, move_metrics, reduce_metrics

log = logging.getLogger(__name__)

T = TypeVar("T")

__all__ = ["BookkeepingMixin"]


class BookkeepingMixin:
    """State lives on the :class:`~olmo_core_b200.train.trainer.Trainer` dataclass that mixes this in."""

    # -- devices, groups, pools ---------------------------------------------------------------------------
    @property
    def bookkeeping_device(self) -> torch.device:
        if self.async_bookkeeping and backend_supports_cpu():
            return torch.device("cpu")
        return self.device

    @property
    def bookkeeping_pg(self) -> Optional[dist.ProcessGroup]:
        return self._bookkeeping_pg

    @property
    def multi_thread_pool(self) -> ThreadPoolExecutor:
        """Pool for work without collectives (uploads, file writes)."""
        if self._multi_thread_pool is None:
            self._multi_thread_pool = ThreadPoolExecutor(max_workers=get_default_thread_count(),
                                                         thread_name_prefix="trainer-mt")
        return self._multi_thread_pool

    @property
    def single_thread_pool(self) -> ThreadPoolExecutor:
        """Pool of exactly one thread: everything that issues bookkeeping collectives goes through it, in order."""
        if self._single_thread_pool is None:
            self._single_thread_pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="trainer-bk")
        return self._single_thread_pool

    # -- metrics --------------------------------------------------------------------------------------------
    def record_metric(self, name: str, value: Union[float, torch.Tensor], reduce_type: Optional[ReduceType] = None,
                      namespace: Optional[str] = None,
                      merge_strategy: MetricMergeStrategy = MetricMergeStrategy.warn) -> None:
        """
        Record a metric for the current step. It stays on its device (no synchronisation) until the window is
        reduced. ``reduce_type`` says how ranks are combined (``None``: rank 0's value is reported).
        """
        if namespace is not None:
            name = f"{namespace.rstrip('/')}/{name.lstrip('/')}"
        value = get_local_tensor(value.detach()).float() if isinstance(value, torch.Tensor) else torch.tensor(float(value))
        step_metrics = self._metrics.setdefault(self.global_step, OrderedDict())
        old = step_metrics.get(name)
        if old is None or merge_strategy == MetricMergeStrategy.latest:
            step_metrics[name] = value
        elif merge_strategy == MetricMergeStrategy.sum:
            step_metrics[name] = old + value.to(old.device)
        elif merge_strategy == MetricMergeStrategy.mean:
            step_metrics[name] = (old + value.to(old.device)) / 2
        elif merge_strategy == MetricMergeStrategy.max:
            step_metrics[name] = torch.max(old, value.to(old.device))
        elif merge_strategy == MetricMergeStrategy.min:
            step_metrics[name] = torch.min(old, value.to(old.device))
        elif merge_strategy == MetricMergeStrategy.warn:
            log.warning(f"Duplicate metric '{name}' recorded for step {self.global_step}; the later value is ignored.")
        elif merge_strategy != MetricMergeStrategy.oldest:
            raise NotImplementedError(merge_strategy)
        known = self._metrics_reduce_type.get(name, reduce_type)
        if name in self._metrics_reduce_type and known != reduce_type:
            raise RuntimeError(f"metric '{name}' was recorded with reduce type '{known}' before, now '{reduce_type}'")
        self._metrics_reduce_type[name] = reduce_type

    def record_ce_loss(self, value: Union[float, torch.Tensor], reduce_type: Optional[ReduceType] = None) -> None:
        self.record_metric(TRAIN_CE_LOSS_METRIC, value, reduce_type=reduce_type)

    def get_metric(self, name: str, namespace: Optional[str] = None) -> Optional[torch.Tensor]:
        """A metric recorded during the current step (reading its value synchronises with the device)."""
        if namespace is not None:
            name = f"{namespace.rstrip('/')}/{name.lstrip('/')}"
        return self._metrics.get(self.global_step, {}).get(name)

    def _log_metrics(self) -> None:
        if not self._metrics:
            return
        # One stacked device->host copy for the whole window; everything after that can run in the background.
        window = move_metrics(self._metrics, self.bookkeeping_device)
        self._metrics.clear()
        if self._metrics_consistent is None:
            self._metrics_consistent = check_metrics_consistent(self._metrics_reduce_type, process_group=self.bookkeeping_pg)
            if not self._metrics_consistent:
                log.warning("Ranks record different sets of metrics (expected e.g. with pipeline parallelism).")
        self.run_bookkeeping_op(reduce_metrics, window, dict(self._metrics_reduce_type), self.bookkeeping_device,
                                process_group=self.bookkeeping_pg, metrics_consistent=bool(self._metrics_consistent),
                                cb=self._check_and_pass_on_metrics)

    def _check_and_pass_on_metrics(self, metrics: Dict[int, Dict[str, float]]) -> None:
        for step in sorted(metrics):
            ce = metrics[step].get(TRAIN_CE_LOSS_METRIC)
            if ce is not None:
                if not math.isfinite(ce):
                    raise RuntimeError(f"{ce} loss encountered at step {step}")
                if ce < 10:
                    metrics[step][TRAIN_PPL_METRIC] = math.exp(ce)
            for cb in self._iter_callbacks():
                cb.pre_log_metrics(step, metrics[step])
            for cb in self._iter_callbacks():
                cb.log_metrics(step, metrics[step])

    # -- background operations ---------------------------------------------------------------------------
    def run_bookkeeping_op(self, op: Callable[..., T], *args, cb: Optional[Callable[[T], None]] = None,
                           op_name: Optional[str] = None, cancel_in_progress: bool = False,
                           allow_multiple: bool = True, distributed: bool = True, **kwargs) -> None:
        """
        Run ``op(*args, **kwargs)`` and then ``cb(result)``. With async bookkeeping the pair runs on a worker thread
        (the single ordered thread when ``distributed``, i.e. when ``op`` may issue collectives); a failure cancels
        the run. ``cancel_in_progress`` drops queued, not yet started operations of the same name;
        ``allow_multiple=False`` skips the call while one of the same name is pending.
        """
        name = op_name or getattr(op, "__qualname__", repr(op))
        if not self.async_bookkeeping or (distributed and is_distributed() and self.bookkeeping_pg is None):
            result = op(*args, **kwargs)
            if cb is not None:
                cb(result)
            return
        pending = self._bookkeeping_queue.setdefault(name, {})
        if cancel_in_progress:
            for key, fut in list(pending.items()):
                if fut.cancel():
                    pending.pop(key, None)
        if not allow_multiple and any(not f.done() for f in pending.values()):
            return

        def task() -> None:
            start = time.perf_counter()
            result = op(*args, **kwargs)
            if cb is not None:
                cb(result)
            took = time.perf_counter() - start
            if took > self.bookkeeping_soft_timeout:
                log.warning(f"Bookkeeping op '{name}' took {took:.1f}s (soft limit {self.bookkeeping_soft_timeout}s)")

        pool = self.single_thread_pool if distributed else self.multi_thread_pool
        key = f"{name}-{time.monotonic_ns()}"
        fut = pool.submit(task)
        pending[key] = fut

        def done(f: Future) -> None:
            pending.pop(key, None)
            if f.cancelled():
                return
            exc = f.exception()
            if exc is not None:
                log.error(f"Bookkeeping op '{name}' failed: {type(exc).__name__}: {exc}")
                self._error = self._error or exc
                self.cancel_run(f"bookkeeping op '{name}' failed: {exc}", no_sync=True)

        fut.add_done_callback(done)

    def _join_bookkeeping_ops(self, timeout: Optional[float] = None) -> None:
        """Wait for queued background operations; re-raises the first failure."""
        deadline = None if timeout is None else time.monotonic() + timeout
        for pending in list(self._bookkeeping_queue.values()):
            for fut in list(pending.values()):
                remaining = None if deadline is None else max(0.0, deadline - time.monotonic())
                try:
                    fut.result(timeout=remaining)
                except Exception:
                    if self._error is not None:
                        raise self._error
                    raise
        if self._error is not None and not self._canceled_error_raised:
            self._canceled_error_raised = True
            raise self._error

    # -- cancellation ----------------------------------------------------------------------------------------
    @property
    def is_canceled(self) -> bool:
        return self._canceled

    def cancel_run(self, reason: str, no_sync: bool = False) -> None:
        """
        Ask for the run to stop. The request becomes effective on all ranks at the next cancellation check
        (every ``cancel_check_interval`` steps); with ``no_sync`` this rank stops at its next check without agreement
        (for failures, where further collectives could hang).
        """
        self._canceling_rank = get_rank()
        self._cancel_reason = reason
        if no_sync:
            self._canceled = True
            log.warning(f"Run canceled from rank {self._canceling_rank}. Reason: {reason}")

    def check_if_canceled(self) -> None:
        """Queue a collective cancellation check (asynchronous when bookkeeping is)."""
        self.run_bookkeeping_op(self._check_if_canceled, op_name="check_if_canceled", cancel_in_progress=True)

    def _check_if_canceled(self) -> None:
        if self._canceled:
            return
        rank = self._canceling_rank if self._canceling_rank is not None else -1
        if is_distributed():
            with cuda_sync_debug_mode(0):
                rank = int(all_reduce_value(rank, self.bookkeeping_device, op=dist.ReduceOp.MAX, group=self.bookkeeping_pg))
                if rank >= 0:
                    reason = broadcast_object(self._cancel_reason, src=rank, group=self.bookkeeping_pg)
                    self._cancel_reason = reason
        if rank >= 0:
            self._canceled = True
            self._canceling_rank = rank
            log.warning(f"Run canceled from rank {rank}. Reason: {self._cancel_reason}")
