"""
The training loop (API and hook order of src/olmo_core/train/trainer.py:100-1560).

``Trainer.fit()``: (optionally) restore a checkpoint, run ``pre_train`` hooks, a dry-run batch, then epochs of
steps. One step is ``pre_load_batch -> next(batch) -> pre_step -> train_batch -> pre_optim_step -> optim_step ->
zero_grads -> post_train_batch -> post_step``; every ``metrics_collect_interval`` steps the recorded metrics are
reduced across ranks and passed to ``log_metrics`` hooks, and every ``cancel_check_interval`` steps ranks agree
on whether the run was canceled. Metrics, cancellation and background work live in
:class:`~olmo_core_b200.train.bookkeeping.BookkeepingMixin`.
"""

from __future__ import annotations

import logging
import signal
import time
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Generator, Iterable, List, Optional, Set, Tuple, Type, TypedDict, Union, cast

import torch
import torch.distributed as dist

from ..aliases import PathOrStr
from ..distributed.utils import (
    backend_supports_cpu,
    barrier,
    broadcast_object,
    get_fs_local_rank,
    get_rank,
    get_world_size,
    is_distributed,
)
from ..exceptions import OLMoConfigurationError
from ..io import copy_dir, copy_file, is_url, join_path, normalize_path
from .bookkeeping import BookkeepingMixin
from .callbacks.callback import Callback
from .checkpoint import Checkpointer
from .common import Duration, DurationUnit, LoadStrategy, ReduceType, StepSkipRange, TrainingProgress
from .train_module import TrainModule
from .utils import EnvRngStates

log = logging.getLogger(__name__)

__all__ = ["Trainer", "TrainerStateDict"]


class TrainerStateDict(TypedDict, total=False):
    global_step: int
    global_train_tokens_seen: int
    global_train_petaflops: float
    max_steps: Optional[int]
    data_loader: Dict[str, Any]
    epoch: int
    world_size: int
    rng: Dict[str, Any]
    callbacks: Dict[str, Dict[str, Any]]


@dataclass
class Trainer(BookkeepingMixin):
    work_dir: Path
    """Local scratch directory (downloads, temporary files)."""
    train_module: TrainModule
    data_loader: Any
    """A :class:`~olmo_core_b200.data.DataLoaderBase`."""
    device: torch.device
    save_folder: str
    """Local directory or URL where checkpoints and other run artefacts go."""
    checkpointer: Checkpointer
    callbacks: Dict[str, Callback]
    max_duration: Duration
    save_overwrite: bool = False
    load_path: Optional[PathOrStr] = None
    """Checkpoint to start from when ``save_folder`` has none."""
    load_strategy: LoadStrategy = LoadStrategy.if_available
    load_trainer_state: Optional[bool] = None
    load_optim_state: Optional[bool] = None
    metrics_collect_interval: int = 5
    dp_process_group: Optional[dist.ProcessGroup] = None
    global_step: int = 0
    global_train_tokens_seen: int = 0
    global_train_petaflops: float = 0.0
    epoch: int = 1
    cancel_check_interval: int = 25
    hard_stop: Optional[Duration] = None
    """Stop (and checkpoint) at this point although ``max_duration``, which shapes the LR schedule, is later."""
    async_bookkeeping: Optional[bool] = None
    bookkeeping_soft_timeout: int = 30
    no_checkpoints: bool = False
    no_evals: bool = False
    steps_to_skip: Optional[List[StepSkipRange]] = None

    _metrics: Dict[int, Dict[str, torch.Tensor]] = field(default_factory=OrderedDict, repr=False)
    _metrics_reduce_type: Dict[str, Optional[ReduceType]] = field(default_factory=dict, repr=False)
    _canceled: bool = False
    _cancel_reason: Optional[str] = None
    _canceling_rank: Optional[int] = None
    _error: Optional[BaseException] = None
    _canceled_error_raised: bool = False
    _rank_batch_size: Optional[int] = None
    _multi_thread_pool: Optional[ThreadPoolExecutor] = field(default=None, repr=False)
    _single_thread_pool: Optional[ThreadPoolExecutor] = field(default=None, repr=False)
    _bookkeeping_queue: Dict[str, Dict[str, Future]] = field(default_factory=dict, repr=False)
    _bookkeeping_pg: Optional[dist.ProcessGroup] = field(default=None, repr=False)
    _blocking_ephemeral_checkpoints: Set[str] = field(default_factory=set, repr=False)
    _checkpoint_loaded: bool = False
    _metrics_consistent: Optional[bool] = None

    def __post_init__(self):
        from .callbacks import CheckpointerCallback, ConsoleLoggerCallback, GarbageCollectorCallback, SpeedMonitorCallback

        self.save_folder = normalize_path(self.save_folder)
        if self.load_path is not None:
            self.load_path = normalize_path(self.load_path)
        if not is_url(self.save_folder) and get_fs_local_rank() != get_rank():
            raise OLMoConfigurationError(
                "Checkpointing to a local directory requires a shared filesystem. If you have one, set the env var "
                "'OLMO_SHARED_FS=1' or set 'FS_LOCAL_RANK' to the global rank of each process."
            )
        if is_url(self.work_dir):
            raise OLMoConfigurationError(f"Trainer working directory must be a local path, got '{self.work_dir}'")
        self.work_dir = Path(normalize_path(self.work_dir))
        if get_fs_local_rank() == 0:
            self.work_dir.mkdir(parents=True, exist_ok=True)
            if not is_url(self.save_folder):
                Path(self.save_folder).mkdir(parents=True, exist_ok=True)

        # callbacks every run needs
        defaults = (
            ("console_logger", ConsoleLoggerCallback, lambda: ConsoleLoggerCallback(metrics_log_interval=self.metrics_collect_interval)),
            ("checkpointer", CheckpointerCallback, CheckpointerCallback),
            ("speed_monitor", SpeedMonitorCallback, SpeedMonitorCallback),
            ("garbage_collector", GarbageCollectorCallback, GarbageCollectorCallback),
        )
        for name, cls, make in defaults:
            if not self.has_callback(cls):
                self.callbacks.setdefault(name, make())
        for cb in self.callbacks.values():
            cb.trainer = self
        self._sort_callbacks()

        if self.dp_process_group is None:
            self.dp_process_group = self.train_module.dp_process_group
        if self._bookkeeping_pg is None and is_distributed():
            if self.async_bookkeeping is None:
                self.async_bookkeeping = backend_supports_cpu()
            if self.async_bookkeeping:
                if not backend_supports_cpu():
                    raise OLMoConfigurationError("A CPU-capable backend is required for async bookkeeping")
                self._bookkeeping_pg = dist.new_group()
        elif self.async_bookkeeping is None:
            self.async_bookkeeping = False

        dl = self.data_loader
        expect = {"dp_world_size": get_world_size(self.dp_process_group), "dp_rank": get_rank(self.dp_process_group),
                  "fs_local_rank": get_fs_local_rank()}
        for attr, want in expect.items():
            got = getattr(dl, attr, want)
            if got != want:
                raise OLMoConfigurationError(f"data loader's '{attr}' is {got}, expected {want}")

        for cb in self.callbacks.values():
            cb.post_attach()
        self.train_module._attach_trainer(self)

    # -- sizes and durations -----------------------------------------------------------------------------------
    @property
    def block_ephemeral_checkpoints(self) -> bool:
        return bool(self._blocking_ephemeral_checkpoints)

    @property
    def global_batch_size(self) -> int:
        """Tokens per step over all data-parallel ranks."""
        return self.data_loader.global_batch_size

    @property
    def rank_batch_size(self) -> int:
        if self._rank_batch_size is None:
            self._rank_batch_size = self.global_batch_size // get_world_size(self.dp_process_group)
        return self._rank_batch_size

    @property
    def tokens_per_batch(self) -> int:
        return self.global_batch_size

    @property
    def steps_per_epoch(self) -> Optional[int]:
        return getattr(self.data_loader, "total_batches", None)

    @property
    def tokens_per_epoch(self) -> Optional[int]:
        steps = self.steps_per_epoch
        return None if steps is None else steps * self.tokens_per_batch

    def _steps_for(self, duration: Duration) -> Optional[int]:
        if duration.unit == DurationUnit.steps:
            return duration.value
        if duration.unit == DurationUnit.epochs:
            steps = self.steps_per_epoch
            return None if steps is None else steps * duration.value
        if duration.unit == DurationUnit.tokens:
            # steps already taken + what the remaining tokens need at the current batch size
            remaining = max(duration.value - self.global_train_tokens_seen, 0)
            return self.global_step + -(-remaining // self.tokens_per_batch)
        raise NotImplementedError(duration.unit)

    def _tokens_for(self, duration: Duration) -> Optional[int]:
        if duration.unit == DurationUnit.tokens:
            return duration.value
        if duration.unit == DurationUnit.steps:
            remaining = max(duration.value - self.global_step, 0)
            return self.global_train_tokens_seen + remaining * self.tokens_per_batch
        if duration.unit == DurationUnit.epochs:
            per_epoch = self.tokens_per_epoch
            return None if per_epoch is None else per_epoch * duration.value
        raise NotImplementedError(duration.unit)

    def convert_duration_to_steps(self, duration: Duration) -> int:
        steps = self._steps_for(duration)
        if steps is None:
            raise RuntimeError("the number of steps in an epoch is unknown for this data loader")
        return steps

    @property
    def max_steps(self) -> Optional[int]:
        return self._steps_for(self.max_duration)

    @property
    def max_tokens(self) -> Optional[int]:
        return self._tokens_for(self.max_duration)

    def _duration_due(self, duration: Duration) -> bool:
        return duration.due(step=self.global_step, tokens=self.global_train_tokens_seen, epoch=self.epoch)

    @property
    def training_complete(self) -> bool:
        if not self._error and self._canceled:
            return True
        if self._duration_due(self.max_duration):
            return True
        return self.hard_stop is not None and self._duration_due(self.hard_stop)

    @property
    def checkpoint_loaded(self) -> bool:
        return self._checkpoint_loaded

    @property
    def training_progress(self) -> TrainingProgress:
        total = self.max_steps
        if self.hard_stop is not None and (hs := self._steps_for(self.hard_stop)) is not None:
            total = hs if total is None else min(total, hs)
        speed = self.callbacks.get("speed_monitor")
        bps = getattr(speed, "bps_avg", None)
        remaining = None
        if bps and total is not None:
            from datetime import timedelta

            remaining = timedelta(seconds=max(total - self.global_step, 0) / bps)
        return TrainingProgress(current_step=self.global_step, total_steps=total, time_remaining=remaining)

    # -- callbacks --------------------------------------------------------------------------------------------
    def get_callback_name(self, callback: Callback) -> str:
        for name, cb in self.callbacks.items():
            if cb is callback:
                return name
        raise KeyError(callback)

    def add_callback(self, name: str, callback: Callback) -> None:
        if name in self.callbacks:
            raise OLMoConfigurationError(f"A callback named '{name}' already exists")
        callback.trainer = self
        self.callbacks[name] = callback
        self._sort_callbacks()
        callback.post_attach()

    def has_callback(self, cb_class: Type[Callback]) -> bool:
        return any(isinstance(cb, cb_class) for cb in self.callbacks.values())

    def _sort_callbacks(self) -> None:
        # (priority desc, name): the same order on every rank, since hooks may issue collectives
        self.callbacks = OrderedDict(sorted(self.callbacks.items(), key=lambda kv: (-kv[1].priority, kv[0])))

    def _iter_callbacks(self) -> Iterable[Callback]:
        return list(self.callbacks.values())

    # -- the loop -------------------------------------------------------------------------------------------------
    def fit(self) -> None:
        """Train until ``max_duration`` (or ``hard_stop``, or cancellation), resuming from a checkpoint if there is one."""
        self._canceled, self._cancel_reason, self._canceling_rank = False, None, None
        if not self.no_checkpoints and not self.checkpoint_loaded and self.load_strategy != LoadStrategy.never:
            # the save folder holds this run's own checkpoints: resume everything from there first
            self.maybe_load_checkpoint(self.save_folder, load_trainer_state=True, load_optim_state=True)
            if self.load_path is not None:
                if not self.checkpoint_loaded:
                    self.maybe_load_checkpoint(self.load_path)
                else:
                    log.warning(f"Ignoring load path ('{self.load_path}') since a checkpoint was found in the save folder")
            if not self.checkpoint_loaded:
                where = f"save folder ('{self.save_folder}') or load path ('{self.load_path}')"
                if self.load_strategy == LoadStrategy.always:
                    raise FileNotFoundError(f"No checkpoint found in {where}")
                log.warning(f"No checkpoint found in {where}, will train from scratch...")
        barrier()
        log.info("Callback order: " + ", ".join(self.callbacks.keys()))
        if self.max_steps is not None:
            log.info(f"Training for {self.max_steps:,d} steps")

        handlers = {}
        try:
            for sig in (signal.SIGTERM, signal.SIGINT):
                handlers[sig] = signal.signal(sig, self._handle_os_signal)
        except ValueError:  # not the main thread: signals stay with whoever owns them
            handlers = {}
        try:
            for cb in self._iter_callbacks():
                cb.pre_train()
            self.train_module.pre_train()
            if self.is_canceled:
                for cb in self._iter_callbacks():
                    cb.post_train()
                self._shutdown()
                return
            if not self.training_complete:
                self._dry_run_batch()
            while not self.training_complete:
                self._fit_epoch()
        except BaseException as exc:
            self._error = exc
            log.error(f"Training failed due to:\n{type(exc).__name__}: {exc}")
            for cb in self._iter_callbacks():
                cb.on_error(exc)
            # no further collectives: ranks may be out of step with each other
            self._shutdown(gracefully=False)
            raise
        finally:
            for sig, old in handlers.items():
                signal.signal(sig, old)
        for cb in self._iter_callbacks():
            cb.post_train()
        self._shutdown()
        log.info("Training complete")

    def _handle_os_signal(self, signalnum, stack_frame) -> None:
        del stack_frame
        name = signal.Signals(signalnum).name
        msg = f"{name} received"
        log.warning(msg)
        self.cancel_run(msg)
        if signalnum == signal.SIGINT:
            raise KeyboardInterrupt

    def _shutdown(self, gracefully: bool = True) -> None:
        if gracefully:
            self._log_metrics()
            self._join_bookkeeping_ops()
        for cb in self._iter_callbacks():
            cb.close()
        for pool in (self._multi_thread_pool, self._single_thread_pool):
            if pool is not None:
                pool.shutdown(wait=gracefully, cancel_futures=not gracefully)
        self._multi_thread_pool = self._single_thread_pool = None
        if gracefully:
            barrier()

    def _iter_batches(self) -> Generator[Dict[str, Any], None, None]:
        it = iter(self.data_loader)
        while True:
            for cb in self._iter_callbacks():
                cb.pre_load_batch()
            try:
                yield next(it)
            except StopIteration:
                return

    def _dry_run_batch(self) -> None:
        """One forward/backward on a mock batch: surfaces out-of-memory and shape errors before real data is touched."""
        try:
            batch = self.data_loader.get_mock_batch()
        except (NotImplementedError, AttributeError):
            return
        log.info("Starting forward/backward dry-run batch...")
        self.train_module.train_batch(batch, dry_run=True)
        self.train_module.zero_grads()
        log.info("Dry-run complete")

    def _should_skip(self) -> bool:
        return any(r.start <= self.global_step < r.stop for r in (self.steps_to_skip or ()))

    def _fit_epoch(self) -> None:
        self.data_loader.reshuffle(self.epoch)
        log.info(f"Starting epoch {self.epoch}...")
        for cb in self._iter_callbacks():
            cb.pre_epoch()
        self.train_module.zero_grads()
        first = True
        for batch in self._iter_batches():
            self.global_step += 1
            n_tokens = self.data_loader.global_num_tokens_in_batch(batch)
            if n_tokens is not None:
                self.global_train_tokens_seen += n_tokens
            n_flops = self.train_module.global_num_flops_in_batch(batch)
            if n_flops is not None:
                self.global_train_petaflops += n_flops / 1e15
            for cb in self._iter_callbacks():
                cb.pre_step(batch)
            if self._should_skip():
                log.warning(f"Skipping training on step {self.global_step:,d} intentionally...")
            else:
                self.train_module.train_batch(batch)
                for cb in self._iter_callbacks():
                    cb.pre_optim_step()
                self.train_module.optim_step()
                self.train_module.zero_grads()
            for cb in self._iter_callbacks():
                cb.post_train_batch()
            for cb in self._iter_callbacks():
                cb.post_step()
            if first or self.global_step % self.metrics_collect_interval == 0:
                self._log_metrics()
            if self.global_step % self.cancel_check_interval == 0:
                self.check_if_canceled()
            first = False
            if self.training_complete:
                self._log_metrics()
                return
        self._log_metrics()
        log.info("Epoch complete")
        for cb in self._iter_callbacks():
            cb.post_epoch()
        self.epoch += 1
        self.data_loader.reset()

    # -- trainer state and checkpoints -------------------------------------------------------------------------
    def state_dict(self) -> TrainerStateDict:
        return {
            "global_step": self.global_step,
            "global_train_tokens_seen": self.global_train_tokens_seen,
            "global_train_petaflops": self.global_train_petaflops,
            "max_steps": self.max_steps,
            "data_loader": self.data_loader.state_dict(),
            "epoch": self.epoch,
            "world_size": get_world_size(),  # the global world size: RNG states are per global rank
            "rng": EnvRngStates.current_state().as_dict(),
            "callbacks": {name: cb.state_dict() for name, cb in self.callbacks.items()},
        }

    def load_state_dict(self, state_dict: TrainerStateDict) -> None:
        """Restore trainer (not model / optimizer) state."""
        sd = cast(Dict[str, Any], state_dict)
        if "data_loader" not in sd and "dataset" in sd:  # older layout
            sd["data_loader"] = sd.pop("dataset")
            sd["data_loader"]["epoch"] = sd["epoch"]
        self.data_loader.load_state_dict(sd["data_loader"])
        self.global_step = sd["global_step"]
        self.global_train_tokens_seen = sd["global_train_tokens_seen"]
        self.global_train_petaflops = sd.get("global_train_petaflops", 0.0)
        self.epoch = sd["epoch"]
        for name, cb_state in sd.get("callbacks", {}).items():
            cb = self.callbacks.get(name)
            if cb is not None:
                cb.load_state_dict(cb_state)
        log.info(f"Will resume training from step {self.global_step}, epoch {self.epoch}")
        if sd.get("world_size") == get_world_size():
            if not EnvRngStates.from_dict(sd["rng"]).restore():
                log.warning("Some RNG states were not restored due to differences in library versions")
        else:
            log.warning("RNG states were saved with a different world size and are not restored.")

    def load_checkpoint(self, dir: PathOrStr, *, load_trainer_state: Optional[bool] = None,
                        load_optim_state: Optional[bool] = None) -> None:
        """Load the checkpoint at ``dir``, or the latest one inside ``dir``."""
        load_trainer_state = self.load_trainer_state if load_trainer_state is None else load_trainer_state
        load_optim_state = self.load_optim_state if load_optim_state is None else load_optim_state
        dir = normalize_path(dir)
        found: Optional[str] = dir
        error: Optional[Exception] = None
        if get_rank() == 0 and not self.checkpointer.dir_is_checkpoint(dir):
            try:
                found = self.checkpointer.latest_checkpoint(dir)
            except FileNotFoundError as e:  # raised on every rank after the broadcast
                found, error = None, e
        found = broadcast_object(found)
        if found is None:
            raise error or FileNotFoundError(f"No checkpoints found in '{dir}'")
        log.info(f"Loading checkpoint from '{found}'...")
        start = time.perf_counter()
        trainer_state = self.checkpointer.load(found, self.train_module, load_trainer_state=load_trainer_state,
                                               load_optim_state=load_optim_state)
        if trainer_state is not None:
            self.load_state_dict(cast(TrainerStateDict, trainer_state))
        self.record_metric("checkpoint/load_duration_s", time.perf_counter() - start, reduce_type=ReduceType.max)
        for cb in self._iter_callbacks():
            cb.post_checkpoint_loaded(found)
        self._checkpoint_loaded = True
        log.info("Checkpoint successfully loaded")

    def maybe_load_checkpoint(self, dir: Optional[PathOrStr] = None, *, load_trainer_state: Optional[bool] = None,
                              load_optim_state: Optional[bool] = None) -> bool:
        """:meth:`load_checkpoint` if ``dir`` has a checkpoint; returns whether one was loaded."""
        dir = self.save_folder if dir is None else dir
        should = self.checkpointer.contains_checkpoint(dir) if get_rank() == 0 else True
        if not broadcast_object(should):
            return False
        self.load_checkpoint(dir, load_trainer_state=load_trainer_state, load_optim_state=load_optim_state)
        return True

    def _checkpoint_path(self) -> str:
        return join_path(self.save_folder, self.checkpointer.checkpoint_dirname(self.global_step))

    def save_checkpoint(self, ephemeral: bool = False) -> PathOrStr:
        """Write a checkpoint for the current step into ``save_folder`` (blocking) and return its path."""
        path = self._checkpoint_path()
        log.info(f"Saving checkpoint for step {self.global_step} to '{path}'...")
        start = time.perf_counter()
        self._log_metrics()
        self._join_bookkeeping_ops()
        self.checkpointer.save(path, self.train_module, cast(Dict[str, Any], self.state_dict()), ephemeral=ephemeral)
        self.record_metric("checkpoint/save_duration_s", time.perf_counter() - start, reduce_type=ReduceType.max)
        for cb in self._iter_callbacks():
            cb.post_checkpoint_saved(path)
        log.info("Checkpoint saved")
        return path

    def save_checkpoint_async(self, ephemeral: bool = False) -> Tuple[PathOrStr, Future]:
        """Like :meth:`save_checkpoint`, returning as soon as the state is staged in host memory."""
        step, path = self.global_step, self._checkpoint_path()
        log.info(f"Saving checkpoint for step {step} to '{path}' asynchronously...")
        start = time.perf_counter()
        self._log_metrics()
        self._join_bookkeeping_ops()
        fut = self.checkpointer.save_async(path, self.train_module, cast(Dict[str, Any], self.state_dict()),
                                           ephemeral=ephemeral)

        def finished(f: Future) -> None:
            f.result()
            self.record_metric("checkpoint/save_async_duration_s", time.perf_counter() - start, reduce_type=ReduceType.max)
            for cb in self._iter_callbacks():
                cb.post_checkpoint_saved(path)
            log.info(f"Checkpoint for step {step} saved successfully")

        fut.add_done_callback(finished)
        return path, fut

    # -- run artefacts ----------------------------------------------------------------------------------------
    def write_file(self, name: str, contents: Union[str, bytes], dir: Optional[PathOrStr] = None) -> PathOrStr:
        """Write a small file into the save folder (or ``dir``). Call from one rank only."""
        return self.checkpointer.write_file(self.save_folder if dir is None else dir, name, contents)

    def persist_working_file(self, name: PathOrStr) -> PathOrStr:
        """Copy ``work_dir/name`` to ``save_folder/name`` (a no-op when they are the same place)."""
        name = Path(name)
        if name.is_absolute():
            name = name.relative_to(self.work_dir)
        source, target = self.work_dir / name, join_path(self.save_folder, name)
        if source.is_file() and str(source) != str(target):
            copy_file(source, target, save_overwrite=self.save_overwrite)
        elif not source.is_file():
            raise FileNotFoundError(source)
        return target

    def persist_working_subdir(self, name: PathOrStr) -> PathOrStr:
        name = Path(name)
        if name.is_absolute():
            name = name.relative_to(self.work_dir)
        source, target = self.work_dir / name, join_path(self.save_folder, name)
        if source.is_dir() and str(source) != str(target):
            copy_dir(source, target, save_overwrite=self.save_overwrite)
        elif not source.is_dir():
            raise FileNotFoundError(source)
        return target
