"""
Weight averaging over the last steps before chosen points of the run
(behaviour of src/olmo_core/train/callbacks/model_merger.py:21-400).

For each merge step ``m`` the parameters of steps ``m - merge_last_n_steps + 1 .. m`` are averaged and written as
a model-only checkpoint ``<save_folder>/step{m}-{output_suffix}/model_and_optim``; evaluator callbacks then run on
the averaged weights (metrics prefixed ``eval/merged``) before the live weights are put back.

The running sums are kept in fp32 on the device that holds the parameter shards: with sharded parameters each rank
accumulates only its own rows, which costs 4 bytes per local parameter per open window and no host traffic.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field
from typing import ClassVar, Dict, List, Optional, Set, Union

import torch

from ...distributed.checkpoint import save_state_dict
from ...distributed.utils import barrier, get_local_tensor, get_rank
from ...exceptions import OLMoConfigurationError
from ...io import clear_directory, dir_is_empty, is_url, join_path
from .callback import Callback
from .checkpointer import CheckpointerCallback

log = logging.getLogger(__name__)

__all__ = ["ModelMergeCallback", "compute_merge_steps_from_decay_schedule", "compute_merge_window_starts"]


@dataclass
class ModelMergeCallback(Callback):
    priority: ClassVar[int] = 2  # before the checkpointer, so that ephemeral saves can be held back in time

    merge_step: Union[int, List[int]] = field(default_factory=list)  # type: ignore[assignment]
    merge_interval: Optional[int] = None
    merge_last_n_steps: int = 500
    output_suffix: str = "merged"
    enabled: bool = False

    _accumulators: Dict[int, Dict[str, torch.Tensor]] = field(default_factory=dict, repr=False)
    _accumulator_counts: Dict[int, int] = field(default_factory=dict, repr=False)
    _merge_steps: List[int] = field(default_factory=list, repr=False)
    _completed_merges: Set[int] = field(default_factory=set, repr=False)

    def __post_init__(self):
        if not self.enabled:
            return
        if self.merge_last_n_steps <= 0:
            raise OLMoConfigurationError(f"merge_last_n_steps must be positive, got {self.merge_last_n_steps}")
        explicit = [self.merge_step] if isinstance(self.merge_step, int) else sorted(self.merge_step)
        explicit = [s for s in explicit if not (isinstance(self.merge_step, int) and s == 0)]
        if self.merge_interval is not None:
            if self.merge_interval <= 0:
                raise OLMoConfigurationError(f"merge_interval must be positive, got {self.merge_interval}")
            if explicit:
                raise OLMoConfigurationError("Cannot set both merge_step and merge_interval; pass all steps as merge_step.")
            return
        if not explicit:
            raise OLMoConfigurationError("Either merge_step or merge_interval must be set.")
        bad = [s for s in explicit if s <= 0]
        if bad:
            raise OLMoConfigurationError(f"merge_step values must be positive, got: {bad}")
        self._merge_steps = explicit

    def _window_start(self, merge_step: int) -> int:
        return max(0, merge_step - self.merge_last_n_steps + 1)

    def _active_windows(self) -> List[int]:
        return [m for m in self._merge_steps if m not in self._completed_merges and self._window_start(m) <= self.step <= m]

    def _merged_checkpoint_path(self, step: int) -> str:
        return str(join_path(self.trainer.save_folder, f"step{step}-{self.output_suffix}"))

    def pre_train(self) -> None:
        if not self.enabled:
            return
        if self.merge_interval is not None:
            max_steps = self.trainer.max_steps
            if max_steps is None:
                raise OLMoConfigurationError("merge_interval requires max_steps to be known; set max_duration on the trainer.")
            self._merge_steps = list(range(self.merge_interval, max_steps + 1, self.merge_interval))
        log.info(f"ModelMergeCallback: merge_steps={self._merge_steps}")
        now = self.step
        for m in self._merge_steps:
            if m < now:
                log.warning(f"Current step {now} is past merge step {m}; this merge is skipped.")
                self._completed_merges.add(m)
            elif self._window_start(m) < now <= m:
                log.warning(f"Resumed at step {now} inside merge window [{self._window_start(m)}, {m}]; the full "
                            f"{self.merge_last_n_steps}-step average cannot be formed and this merge is skipped.")
                self._completed_merges.add(m)
        remaining = [m for m in self._merge_steps if m not in self._completed_merges]
        for m in remaining:
            if m < self.merge_last_n_steps:
                raise OLMoConfigurationError(f"Merge step {m} is less than merge_last_n_steps ({self.merge_last_n_steps}).")
        ckpt = next((cb for cb in self.trainer.callbacks.values() if isinstance(cb, CheckpointerCallback)), None)
        if ckpt is not None and ckpt.save_interval:
            for m in remaining:
                start = self._window_start(m)
                first = (start // ckpt.save_interval + 1) * ckpt.save_interval
                if start < first < m:
                    log.warning(f"Permanent checkpoint at step {first} falls inside merge window [{start}, {m}]; "
                                "resuming from it would skip this merge.")

    def _local_params(self) -> Dict[str, torch.Tensor]:
        return {n: get_local_tensor(p.data) for n, p in self.trainer.train_module.model.named_parameters()}

    @torch.no_grad()
    def post_train_batch(self) -> None:
        if not self.enabled:
            return
        active = self._active_windows()
        if not active:
            self.unblock_ephemeral_checkpoints()
            return
        params = self._local_params()
        for m in active:
            acc = self._accumulators.get(m)
            if acc is None:
                log.info(f"Starting weight accumulation for merge step {m} at step {self.step}")
                acc = self._accumulators[m] = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in params.items()}
                self._accumulator_counts[m] = 0
            torch._foreach_add_(list(acc.values()), [p.float() for p in params.values()])
            self._accumulator_counts[m] += 1
        for m in active:
            if self.step == m:
                self._save_merged_checkpoint(m)
        if any(m not in self._completed_merges for m in active):
            self.block_ephemeral_checkpoints()  # a resume from inside the window could not complete the average
        else:
            self.unblock_ephemeral_checkpoints()

    @torch.no_grad()
    def _save_merged_checkpoint(self, merge_step: int) -> None:
        acc, count = self._accumulators.get(merge_step), self._accumulator_counts.get(merge_step, 0)
        if acc is None or count == 0:
            log.warning(f"No weights accumulated for merge step {merge_step}, cannot save")
            return
        log.info(f"Saving merged checkpoint (average of {count} steps) at step {merge_step}")
        out = self._merged_checkpoint_path(merge_step)
        if get_rank() == 0:
            if not dir_is_empty(out):
                clear_directory(out)
            if not is_url(out):
                os.makedirs(out, exist_ok=True)
        barrier()
        tm = self.trainer.train_module
        params = self._local_params()
        live = {n: p.clone() for n, p in params.items()}
        for n, p in params.items():
            p.copy_((acc[n] / count).to(p.dtype))
        runtime = getattr(tm, "runtime", None)
        if runtime is not None:
            runtime.sync_lowp()
        barrier()
        try:
            save_state_dict(join_path(out, "model_and_optim"), tm.state_dict_to_save(optim=False),
                            process_group=self.trainer.checkpointer.process_group, save_overwrite=True)
            barrier()
            log.info(f"Merged checkpoint saved to: {out}")
            self._evaluate_merged()
        finally:
            for n, p in params.items():
                p.copy_(live[n])
            if runtime is not None:
                runtime.sync_lowp()
            barrier()
        del self._accumulators[merge_step], self._accumulator_counts[merge_step]
        self._completed_merges.add(merge_step)

    def _evaluate_merged(self) -> None:
        from .evaluator_callback import EvaluatorCallback

        evaluators = [cb for cb in self.trainer.callbacks.values() if isinstance(cb, EvaluatorCallback)]
        if not evaluators:
            log.info("No EvaluatorCallback found, skipping merged model evaluation")
        for cb in evaluators:
            cb.perform_eval(prefix="eval/merged")


def compute_merge_steps_from_decay_schedule(period_lengths: List[int], tokens_per_step: int, decay: Optional[int] = None,
                                            decay_fraction: Optional[float] = None) -> List[int]:
    """The last step before the LR decay of each period (lengths and ``decay`` in tokens): where merging pays most."""
    if decay is None and decay_fraction is None:
        raise ValueError("Either decay or decay_fraction must be set")
    steps, total = [], 0
    for length in period_lengths:
        total += length
        decay_tokens = decay if decay is not None else int(round(decay_fraction * length))  # type: ignore[operator]
        steps.append((total - decay_tokens) // tokens_per_step)
    return steps


def compute_merge_window_starts(merge_steps: List[int], merge_last_n_steps: int) -> List[int]:
    """
    Steps at which a checkpoint should exist (pass as the checkpointer's ``fixed_steps``) so that every merge window
    can be re-run from its beginning after an interruption. Overlapping windows share their earliest start.
    """
    starts: List[int] = []
    prev = -1
    for m in sorted(merge_steps):
        start = max(0, m - merge_last_n_steps + 1)
        if start > prev:
            starts.append(start)
        prev = m
    return starts
