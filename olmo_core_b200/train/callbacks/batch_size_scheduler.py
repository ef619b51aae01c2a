"""
Batch-size schedule with square-root learning-rate scaling
(behaviour of src/olmo_core/train/callbacks/batch_size_scheduler.py:22-190).

``schedule[i]`` says when ``batch_sizes[i]`` (tokens per step) takes effect; the first entry must be at 0 and every
change must be by an integer factor. When the batch size changes by a factor ``r`` the base learning rate of every
parameter group is multiplied by ``sqrt(r)`` -- the scaling rule under which Adam's update statistics are preserved.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass, field
from typing import List

from ...exceptions import OLMoConfigurationError
from ..common import Duration
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["BatchSizeSchedulerCallback"]


@dataclass
class BatchSizeSchedulerCallback(Callback):
    batch_sizes: List[int] = field(default_factory=list)
    schedule: List[Duration] = field(default_factory=list)
    enabled: bool = True

    def __post_init__(self):
        if len(self.batch_sizes) != len(self.schedule):
            raise OLMoConfigurationError("batch_sizes and schedules should have the same number of items")
        if not self.schedule or not self.enabled:
            return
        if len({d.unit for d in self.schedule}) > 1:
            raise OLMoConfigurationError("batch size scheduler must use consistent units for all points in the schedule")
        if self.schedule[0].value != 0:
            raise OLMoConfigurationError("batch size schedule must start at 0")
        for (prev_bs, prev_at), (bs, at) in zip(zip(self.batch_sizes, self.schedule),
                                                zip(self.batch_sizes[1:], self.schedule[1:])):
            if at.value <= prev_at.value:
                raise OLMoConfigurationError("events in the batch size schedule must be in increasing order")
            if bs == prev_bs:
                raise OLMoConfigurationError("invalid batch size schedule, duplicate batch size in schedule")
            big, small = max(bs, prev_bs), min(bs, prev_bs)
            if big % small != 0:
                raise OLMoConfigurationError("invalid batch size schedule, batch size can only change by an integer factor")

    @property
    def current_batch_size(self) -> int:
        return self.trainer.data_loader.global_batch_size

    def _schedulers_and_optims(self):
        tm = self.trainer.train_module
        optims = getattr(tm, "optimizers", None) or ([tm.optim] if hasattr(tm, "optim") else [])
        return getattr(tm, "scheduler", None), optims

    def post_attach(self) -> None:
        if not self.schedule:
            return
        from ...optim.scheduler import WSD, ConstantScheduler

        scheduler, _ = self._schedulers_and_optims()
        # The end point of the LR schedule must not move when the number of tokens per step changes.
        if (scheduler is not None and not isinstance(scheduler, (ConstantScheduler, WSD))
                and getattr(scheduler, "t_max", None) is None and self.trainer.max_duration.unit != "steps"
                and getattr(scheduler, "units", None) != "tokens"):
            raise OLMoConfigurationError(
                f"Batch size scheduler requires the {scheduler.__class__.__name__} LR scheduler's units to be set to "
                "'tokens' unless 't_max' is set."
            )
        self._maybe_update()

    def post_checkpoint_loaded(self, *args) -> None:
        del args
        self._maybe_update()  # base learning rates come from the config after a restore, not from the checkpoint

    def pre_load_batch(self) -> None:
        self._maybe_update()

    def post_step(self) -> None:
        self.trainer.record_metric("train/global batch size", self.current_batch_size)

    def _maybe_update(self) -> None:
        if not self.enabled:
            return
        t = self.trainer
        for target, start in reversed(list(zip(self.batch_sizes, self.schedule))):
            if not start.due(step=t.global_step, tokens=t.global_train_tokens_seen, epoch=t.epoch):
                continue
            cur = self.current_batch_size
            if target > cur:
                # grow only on a boundary of the larger batches so that no instance is skipped or repeated
                if t.data_loader.batches_processed % (target // cur) == 0:
                    self._apply(target)
            elif target < cur:
                self._apply(target)
            break

    def _apply(self, batch_size: int) -> None:
        log.info(f"Changing global batch size to {batch_size:,d}...")
        factor = math.sqrt(batch_size / self.current_batch_size)
        self.trainer.data_loader.global_batch_size = batch_size
        scheduler, optims = self._schedulers_and_optims()
        if not optims:
            raise NotImplementedError(f"Unable to adjust learning rate for {type(self.trainer.train_module).__name__}")
        lr_field = getattr(scheduler, "lr_field", "lr")
        initial_field = getattr(scheduler, "initial_lr_field", "initial_lr")
        for optim in optims:
            for group in optim.param_groups:
                key = initial_field if (scheduler is not None and initial_field in group) else lr_field
                group[key] = group[key] * factor
                if scheduler is None or key == lr_field:
                    continue
                # the visible learning rate follows at the next scheduler update; keep it consistent meanwhile
                value = group[lr_field]
                group[lr_field] = value * factor if not hasattr(value, "mul_") else value.mul_(factor)
        self.trainer._rank_batch_size = None
