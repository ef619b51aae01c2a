"""
Checkpoint scheduling (options and behaviour of src/olmo_core/train/callbacks/checkpointer.py:27-330).

Two kinds of checkpoints are written into the trainer's save folder: *permanent* ones every ``save_interval``
steps (and at ``fixed_steps``, before training and after it), of which at most ``max_checkpoints`` are kept, and
*ephemeral* ones every ``ephemeral_save_interval`` steps, of which only the newest survives. Removal happens
after the next checkpoint is complete, never before.
"""

from __future__ import annotations

import logging
from concurrent.futures import Future
from dataclasses import dataclass, field
from datetime import timedelta
from typing import ClassVar, List, Optional, Tuple

import torch.distributed as dist

from ...config import StrEnum
from ...distributed.utils import backend_supports_cpu, broadcast_object, get_fs_local_rank, get_rank, is_distributed
from ...exceptions import OLMoConfigurationError
from ...io import clear_directory, is_url, join_path, remove_file
from ...utils import wait_for
from ..checkpoint import Checkpointer
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["CheckpointerCallback", "CheckpointRemovalStrategy"]


class CheckpointRemovalStrategy(StrEnum):
    ephemeral_only = "ephemeral_only"
    """Of the checkpoints left by earlier runs, remove those at multiples of ``ephemeral_save_interval``."""
    all_non_permanent = "all_non_permanent"
    """Remove every earlier checkpoint that is not at a multiple of ``save_interval`` or a fixed step."""
    never = "never"


@dataclass
class CheckpointerCallback(Callback):
    priority: ClassVar[int] = 1

    save_interval: Optional[int] = 250
    ephemeral_save_interval: Optional[int] = None
    pre_train_checkpoint: Optional[bool] = None
    save_async: Optional[bool] = None
    remove: CheckpointRemovalStrategy = CheckpointRemovalStrategy.ephemeral_only
    ephemeral_cooldown: Optional[int] = None
    """Minimum number of steps between any checkpoint and the next ephemeral one."""
    fixed_steps: Optional[List[int]] = None
    max_checkpoints: Optional[int] = 3
    """How many permanent checkpoints written by this run to keep (None: all)."""
    enabled: bool = True

    _future: Optional[Future] = field(default=None, repr=False)
    _latest_checkpoint_step: int = -1
    _latest_checkpoint_path: str = ""
    _checkpoints: List[str] = field(default_factory=list)
    _ephemeral_checkpoints: List[str] = field(default_factory=list)
    _checkpoints_to_remove: List[str] = field(default_factory=list)

    def __post_init__(self):
        if self.save_interval is not None and self.save_interval < 1:
            raise OLMoConfigurationError("'save_interval' must be at least 1")
        if self.ephemeral_save_interval is not None:
            if self.ephemeral_save_interval < 1:
                raise OLMoConfigurationError("'ephemeral_save_interval' must be at least 1")
            if self.save_interval is not None and self.ephemeral_save_interval >= self.save_interval:
                raise OLMoConfigurationError("'ephemeral_save_interval' must be less than 'save_interval'")
        if self.max_checkpoints is not None and self.max_checkpoints < 1:
            raise OLMoConfigurationError("'max_checkpoints' must be at least 1")

    # -- helpers ------------------------------------------------------------------------------------------
    @property
    def checkpointer(self) -> Checkpointer:
        return self.trainer.checkpointer

    @property
    def save_folder(self) -> str:
        return self.trainer.save_folder

    @property
    def checkpoint_pending(self) -> bool:
        return self._future is not None

    def _await_last_checkpoint(self, blocking: bool = True) -> Optional[Future]:
        fut = self._future
        if fut is None or not (blocking or fut.done()):
            return None
        fut.result()
        if get_rank() == 0:
            wait_for(lambda: self.checkpointer.dir_is_checkpoint(self._latest_checkpoint_path),
                     "the checkpoint to be finalized", timeout=self.checkpointer.FS_TIMEOUT)
        self._future = None
        return fut

    def _save(self, save_async: Optional[bool] = None, ephemeral: bool = False) -> str:
        save_async = self.save_async if save_async is None else save_async
        self._await_last_checkpoint()
        if save_async:
            path, self._future = self.trainer.save_checkpoint_async(ephemeral=ephemeral)
        else:
            path = self.trainer.save_checkpoint(ephemeral=ephemeral)
        self._latest_checkpoint_step, self._latest_checkpoint_path = self.step, str(path)
        return str(path)

    def _save_permanent(self, save_async: Optional[bool] = None) -> None:
        self._checkpoints.append(self._save(save_async=save_async))
        if self.max_checkpoints is not None:
            while len(self._checkpoints) > self.max_checkpoints:
                self._checkpoints_to_remove.append(self._checkpoints.pop(0))

    def _remove(self, path: str) -> None:
        log.info(f"Removing old checkpoint at '{path}'...")
        if get_rank() == 0:  # drop the completion marker first so that nobody picks up a half-deleted checkpoint
            try:
                remove_file(join_path(path, self.checkpointer.METADATA_FNAME))
            except FileNotFoundError:
                pass
        if (is_url(path) and get_rank() == 0) or (not is_url(path) and get_fs_local_rank() == 0):
            self.trainer.run_bookkeeping_op(clear_directory, path, op_name=f"clear_directory {path}", distributed=False)

    def _flush_removals(self) -> None:
        for path in self._checkpoints_to_remove:
            self._remove(path)
        self._checkpoints_to_remove.clear()

    def _leftovers(self) -> List[Tuple[int, str]]:
        """Checkpoints of earlier runs in the save folder that this run is allowed to delete."""
        found: List[Tuple[int, str]] = []
        try:
            for step, path in self.checkpointer.find_checkpoints(self.save_folder):
                permanent = (step == 0 or step > self.step or (self.fixed_steps is not None and step in self.fixed_steps)
                             or (self.save_interval is not None and step % self.save_interval == 0))
                if permanent:
                    continue
                if self.remove == CheckpointRemovalStrategy.all_non_permanent or (
                    self.ephemeral_save_interval is not None and step % self.ephemeral_save_interval == 0
                ):
                    found.append((step, path))
        except FileNotFoundError:
            pass
        return found

    # -- hooks ----------------------------------------------------------------------------------------------
    def pre_train(self) -> None:
        if not self.enabled:
            return
        if self.save_async is None:
            self.save_async = backend_supports_cpu()
        if is_distributed() and self.save_async and self.checkpointer.process_group is None:
            if not backend_supports_cpu():
                raise RuntimeError("a CPU-capable backend is required for async checkpointing")
            log.info("Creating a process group for asynchronous checkpointing")
            self.checkpointer.process_group = dist.new_group(timeout=timedelta(minutes=30))
        if self.step == 0 and (self.pre_train_checkpoint or (self.pre_train_checkpoint is None and not self.trainer.checkpoint_loaded)):
            self._checkpoints.append(self._save())
        if self.remove != CheckpointRemovalStrategy.never:
            leftovers = self._leftovers() if get_rank() == 0 else []  # one rank lists the (possibly remote) folder
            leftovers = broadcast_object(leftovers)
            self._ephemeral_checkpoints = [p for _, p in sorted(leftovers)]
            for p in self._ephemeral_checkpoints:
                log.info(f"Found ephemeral checkpoint '{p}'; it will be removed after the next checkpoint is saved")

    def post_train_batch(self) -> None:
        if not self.enabled:
            return
        self._await_last_checkpoint(blocking=False)
        if not self.checkpoint_pending:
            self._flush_removals()
        if (self.fixed_steps is not None and self.step in self.fixed_steps) or (
            self.save_interval is not None and self.step % self.save_interval == 0
        ):
            self._save_permanent()
        elif (self.ephemeral_save_interval is not None and self.step % self.ephemeral_save_interval == 0
              and not self.trainer.block_ephemeral_checkpoints):
            if self.ephemeral_cooldown is not None and self.step - self._latest_checkpoint_step < self.ephemeral_cooldown:
                return
            self._ephemeral_checkpoints.append(self._save(ephemeral=True))
            while len(self._ephemeral_checkpoints) > 1:
                self._checkpoints_to_remove.append(self._ephemeral_checkpoints.pop(0))

    def post_train(self) -> None:
        if not self.enabled:
            return
        if self.step > self._latest_checkpoint_step:
            self._save_permanent(save_async=False)
        self._await_last_checkpoint()
        self._flush_removals()
