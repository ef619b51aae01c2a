"""
The model ladder itself and the two strategy interfaces it is parameterised by
(API of src/olmo_core/model_ladder/base.py:48-742).

* :class:`ModelConfigurator` answers model-shaped questions for a size label ("190M"): the model config, the per-device
  micro-batch, the smallest device mesh and how to build the train module.
* :class:`RunConfigurator` answers run-shaped questions for a parameter count: batch size, duration, optimizer,
  schedule and the checkpoints worth keeping.
* :class:`ModelLadder` combines both with data sources and a directory layout (``<dir>/<size>/step<N>``), chooses the
  number of devices (as many multiples of the minimal mesh as the batch size can feed), and runs / inspects the rungs.
"""

from __future__ import annotations

import concurrent.futures
import json
import logging
import math
import typing
from abc import ABCMeta, abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, Generic, List, NamedTuple, Optional, Tuple, TypeVar

from .. import io
from ..aliases import PathOrStr
from ..config import Config
from ..data import DataMix, NumpyPaddedFSLDatasetConfig, TokenizerConfig
from ..distributed import utils as dist_utils
from ..exceptions import OLMoConfigurationError
from ..optim import OptimConfig, Scheduler
from ..train import (
    Duration,
    DurationUnit,
    TrainerConfig,
    callbacks,
    prepare_training_environment,
    teardown_training_environment,
)
from ..train.checkpoint import Checkpointer
from ..train.train_module import TrainModule
from ..utils import warn_once
from .utils import format_count, format_tokens

log = logging.getLogger(__name__)

__all__ = ["DeviceMeshSpec", "RunCheckpointInfo", "ModelConfigurator", "RunConfigurator", "ModelLadder"]

M = TypeVar("M")


class DeviceMeshSpec(NamedTuple):
    world_size: int
    dp_world_size: Optional[int]  # smallest data-parallel group; ``None`` means the whole world


@dataclass(frozen=True)
class RunCheckpointInfo:
    name: str
    step: int
    tokens: int
    path: PathOrStr
    metrics_path: Optional[PathOrStr]
    exists: bool

    def display(self) -> str:
        head = f"Step {self.step:,d} ({format_tokens(self.tokens)}) [b cyan]{self.name}[/]"
        if not self.exists:
            return f"[b yellow]✘[/] {head}"
        text = f"[b green]✔[/] {head}\n  ↳ checkpoint: [u blue]{self.path}[/]"
        if self.metrics_path is not None:
            text += f"\n  ↳ metrics:    [u blue]{self.metrics_path}[/]"
        return text


@dataclass(kw_only=True)
class ModelConfigurator(Config, Generic[M], metaclass=ABCMeta):
    @abstractmethod
    def configure_model(self, *, size_spec: str, sequence_length: int, tokenizer: TokenizerConfig, device_type: str) -> M:
        raise NotImplementedError

    @abstractmethod
    def configure_rank_microbatch_size(self, *, size_spec: str, sequence_length: int, device_type: str) -> int:
        raise NotImplementedError

    @abstractmethod
    def configure_minimal_device_mesh_spec(self, *, size_spec: str, sequence_length: int, device_type: str) -> DeviceMeshSpec:
        raise NotImplementedError

    @abstractmethod
    def build_train_module(self, *, size_spec: str, sequence_length: int, rank_microbatch_size: int, model_config: M,
                           optim_config: OptimConfig, scheduler: Scheduler, device_type: str) -> TrainModule:
        raise NotImplementedError


@dataclass(kw_only=True)
class RunConfigurator(Config, metaclass=ABCMeta):
    @abstractmethod
    def configure_target_batch_size(self, num_params: int) -> int:
        """Target global batch in tokens; the ladder rounds it to what the device mesh can divide."""
        raise NotImplementedError

    @abstractmethod
    def configure_duration(self, num_params: int, batch_size: int) -> Duration:
        raise NotImplementedError

    @abstractmethod
    def configure_optimizer(self, num_params: int, batch_size: int) -> OptimConfig:
        raise NotImplementedError

    @abstractmethod
    def configure_lr_scheduler(self, num_params: int, batch_size: int) -> Scheduler:
        raise NotImplementedError

    @abstractmethod
    def configure_checkpoint_intervals(self, num_params: int, batch_size: int) -> List[Tuple[Duration, str]]:
        """(when, description) of every checkpoint to keep."""
        raise NotImplementedError

    @abstractmethod
    def plot_lr_schedule(self, num_params: int, batch_size: int, *, show: bool = True,
                         save_path: Optional[PathOrStr] = None) -> Optional[PathOrStr]:
        raise NotImplementedError


@dataclass(kw_only=True)
class ModelLadder(Config):
    name: str
    dir: str  # root of the results; one sub-folder per size
    sizes: List[str]
    max_devices: int
    device_type: str
    model_configurator: ModelConfigurator
    run_configurator: RunConfigurator
    data_loader: Any  # composable data loader config
    instance_sources: List[Any]  # instance source configs
    tokenizer: TokenizerConfig
    project: Optional[str] = None
    sequence_length: int = 8192
    seed: int = 42
    backend: str = "cpu:gloo,cuda:nccl"

    def __post_init__(self):
        if self.max_devices <= 0:
            raise OLMoConfigurationError("max_devices must be a positive integer.")
        for size in self.sizes:
            needed = self._mesh_spec(size).world_size
            if needed > self.max_devices:
                raise OLMoConfigurationError(f"Model of size {size} requires at least {needed} devices, "
                                             f"but max_devices is set to {self.max_devices}.")

    # -- small accessors -----------------------------------------------------------------------------------
    @property
    def work_dir(self) -> PathOrStr:
        return "./cache" if io.is_url(self.dir) else str(io.join_path(self.dir, "cache"))

    def _mesh_spec(self, size_spec: str) -> DeviceMeshSpec:
        return self.model_configurator.configure_minimal_device_mesh_spec(
            size_spec=size_spec, sequence_length=self.sequence_length, device_type=self.device_type)

    def _require(self, size_spec: str) -> None:
        if size_spec not in self.sizes:
            raise ValueError(f"Invalid size_spec '{size_spec}', must be one of {self.sizes}")

    def get_model_config(self, size_spec: str):
        return self.model_configurator.configure_model(size_spec=size_spec, sequence_length=self.sequence_length,
                                                       tokenizer=self.tokenizer, device_type=self.device_type)

    def get_num_params(self, size_spec: str) -> int:
        return self.get_model_config(size_spec).num_non_embedding_params

    def get_num_devices(self, size_spec: str) -> int:
        return self._configure_batch_size_and_num_devices(size_spec, self.get_num_params(size_spec))[2]

    def get_save_folder(self, size_spec: str) -> str:
        return str(io.join_path(self.dir, size_spec))

    # -- planning ------------------------------------------------------------------------------------------
    def _configure_batch_size_and_num_devices(self, size_spec: str, num_params: int) -> Tuple[int, int, int, int]:
        """→ (global batch in tokens, micro-batch per device in tokens, devices, data-parallel world size)."""
        target = self.run_configurator.configure_target_batch_size(num_params)
        micro = self.model_configurator.configure_rank_microbatch_size(
            size_spec=size_spec, sequence_length=self.sequence_length, device_type=self.device_type)
        micro = min(micro, target)
        min_world, min_dp = self._mesh_spec(size_spec)
        min_dp = min_world if min_dp is None else min_dp
        if min_world % min_dp != 0:
            raise OLMoConfigurationError(f"Invalid device mesh spec for model of size '{size_spec}': minimum world size "
                                         f"{min_world} is not divisible by the minimum data parallel world size {min_dp}.")
        if self.max_devices < min_world:
            raise OLMoConfigurationError(f"Not enough devices ({self.max_devices}) to run model of size '{size_spec}' "
                                         f"which requires at least {min_world} devices.")
        # one "unit" = the tokens the minimal mesh consumes per micro-step; the batch is a whole number of units, and the
        # mesh is replicated while every replica still has at least one unit to work on
        unit = micro * min_dp
        units = max(1, round(target / unit))
        replicas = min(self.max_devices // min_world, units)
        devices, dp = min_world * replicas, min_dp * replicas
        per_step = micro * dp
        batch = max(1, round(units * unit / per_step)) * per_step
        off = abs(batch - target) / target
        if off > 0.1:
            msg = (f"Global batch size to use ({format_tokens(batch)}) differs from target global batch size "
                   f"({format_tokens(target)}) by ~{100 * off:.1f}%.")
            if micro // self.sequence_length > 1:
                msg += ("\nConsider decreasing the configured rank micro-batch size, which is set by the method "
                        f"{type(self.model_configurator).__name__}.configure_rank_microbatch_size().")
            warn_once(msg, UserWarning)
        return batch, micro, devices, dp

    def _duration_to_steps(self, d: Duration, global_batch_size: int) -> int:
        if d.unit == DurationUnit.steps:
            return d.value
        if d.unit == DurationUnit.tokens:
            return d.value // global_batch_size
        raise ValueError(f"Unsupported checkpoint interval duration unit: {d.unit}.")

    def _get_checkpoint_intervals(self, *, num_params: int, global_batch_size: int) -> List[int]:
        return [self._duration_to_steps(d, global_batch_size)
                for d, _ in self.run_configurator.configure_checkpoint_intervals(num_params, global_batch_size)]

    def dry_run(self, size_spec: str, show_plot: bool = True, save_plot: Optional[PathOrStr] = None) -> Dict[str, int]:
        """Print (and return) the plan for one rung; optionally plot its learning-rate schedule."""
        self._require(size_spec)
        n = self.get_num_params(size_spec)
        target = self.run_configurator.configure_target_batch_size(n)
        batch, micro, devices, dp = self._configure_batch_size_and_num_devices(size_spec, n)
        assert micro % self.sequence_length == 0 and batch % (micro * dp) == 0
        plan = {"num_params": n, "target_batch_size": target, "global_batch_size": batch, "rank_microbatch_size": micro,
                "num_devices": devices, "dp_world_size": dp, "grad_accum_steps": batch // (micro * dp)}
        print(f"Dry run for model size {size_spec}:\n"
              f" > Actual number of non-embedding params is {format_count(n)}\n"
              f" > Target batch size is {target:,d} tokens\n"
              f" > Actual batch size is {batch:,d} tokens, which is {batch // self.sequence_length:,d} instance(s)\n"
              f" > Micro-batch size per device is {micro:,d} tokens, which is {micro // self.sequence_length} instance(s)\n"
              f" > The run requires {devices} out of {self.max_devices} devices, with a data-parallel world size of {dp:,d}\n"
              f" > So there will be {plan['grad_accum_steps']:,d} grad accumulation step(s) per batch")
        if show_plot or save_plot is not None:
            path = self.run_configurator.plot_lr_schedule(n, batch, show=show_plot, save_path=save_plot)
            if path is not None:
                log.info("Saved LR schedule plot to '%s'", path)
        return plan

    # -- running -------------------------------------------------------------------------------------------
    def _get_mix_base_dir(self) -> str:
        from ..internal.common import get_root_dir

        return get_root_dir("local")

    def _get_in_loop_eval_tasks(self) -> List[str]:
        from ..eval.task_groups import TASK_GROUPS

        return sorted(TASK_GROUPS.get("fast", []))

    def _configure_trainer(self, size_spec: str, for_benchmarking: bool = False) -> TrainerConfig:
        run_name = f"{self.name}-{size_spec}"
        n = self.get_num_params(size_spec)
        batch = self._configure_batch_size_and_num_devices(size_spec, n)[0]
        cbs: Dict[str, Any] = {
            "gpu_monitor": callbacks.GPUMemoryMonitorCallback(),
            "config_saver": callbacks.ConfigSaverCallback(),
            "garbage_collector": callbacks.GarbageCollectorCallback(),
            "checkpointer": callbacks.CheckpointerCallback(
                ephemeral_save_interval=1000, ephemeral_cooldown=250, save_interval=None, save_async=True,
                fixed_steps=self._get_checkpoint_intervals(num_params=n, global_batch_size=batch),
                enabled=not for_benchmarking),
            "profiler": callbacks.ProfilerCallback(enabled=for_benchmarking),
            "gap_monitor": callbacks.GAPMonitorCallback(enabled=False, interval=10),
            "slack_notifier": callbacks.SlackNotifierCallback(name=run_name, enabled=False),
            "beaker": callbacks.BeakerCallback(),
            "wandb": callbacks.WandBCallback(name=run_name, group=self.name, project=self.project or self.name,
                                             cancel_check_interval=50, enabled=not for_benchmarking),
            "lm_evaluator": callbacks.LMEvaluatorCallbackConfig(
                eval_dataset=NumpyPaddedFSLDatasetConfig.from_data_mix(
                    DataMix.v3_small_ppl_validation, mix_base_dir=self._get_mix_base_dir(),
                    sequence_length=self.sequence_length, tokenizer=self.tokenizer, work_dir=str(self.work_dir)),
                eval_interval=None, eval_on_checkpoint=True, enabled=not for_benchmarking),
        }
        tasks = self._get_in_loop_eval_tasks()
        if tasks:
            cbs["downstream_evaluator"] = callbacks.DownstreamEvaluatorCallbackConfig(
                tasks=tasks, tokenizer=self.tokenizer, eval_interval=None, eval_on_checkpoint=True,
                enabled=not for_benchmarking)
        return TrainerConfig(
            save_folder=self.get_save_folder(size_spec), work_dir=str(self.work_dir), metrics_collect_interval=10,
            cancel_check_interval=10, max_duration=self.run_configurator.configure_duration(n, batch),
            hard_stop=Duration.steps(100) if for_benchmarking else None, no_checkpoints=for_benchmarking,
            no_evals=for_benchmarking, save_overwrite=True, callbacks=cbs)

    def run(self, size_spec: str, for_benchmarking: bool = False) -> None:
        """Train one rung here, on the ranks of the current job."""
        self._require(size_spec)
        prepare_training_environment(seed=self.seed, backend=self.backend)
        try:
            from ..data.composable.utils import set_composable_seed

            set_composable_seed(self.seed)
        except ImportError:
            pass
        model_config = self.get_model_config(size_spec)
        n = model_config.num_non_embedding_params
        batch, micro, devices, _ = self._configure_batch_size_and_num_devices(size_spec, n)
        if devices != dist_utils.get_world_size():
            raise OLMoConfigurationError(f"Requested {devices} devices for model of size '{size_spec}', "
                                         f"but {dist_utils.get_world_size()} are available.")
        optim = self.run_configurator.configure_optimizer(n, batch)
        scheduler = self.run_configurator.configure_lr_scheduler(n, batch)
        trainer_config = self._configure_trainer(size_spec, for_benchmarking=for_benchmarking)
        sources = [s.build(work_dir=self.work_dir) for s in self.instance_sources]
        loader = self.data_loader.build(*sources, work_dir=self.work_dir, global_batch_size=batch, tokenizer=self.tokenizer)
        if loader.sequence_length != self.sequence_length:
            raise OLMoConfigurationError(f"Data loader sequence of {loader.sequence_length} does not match configured "
                                         f"sequence length of {self.sequence_length}.")
        train_module = self.model_configurator.build_train_module(
            size_spec=size_spec, sequence_length=self.sequence_length, rank_microbatch_size=micro,
            model_config=model_config, optim_config=optim, scheduler=scheduler, device_type=self.device_type)
        trainer = trainer_config.build(train_module, loader)
        typing.cast(callbacks.ConfigSaverCallback, trainer.callbacks["config_saver"]).config = {
            "seed": self.seed, "size": str(size_spec), "model": model_config.as_config_dict(),
            "optim": optim.as_config_dict(), "scheduler": scheduler.as_config_dict(),
            "data_loader": self.data_loader.as_config_dict(),
            "instance_sources": [s.as_config_dict() for s in self.instance_sources]}
        trainer.fit()
        teardown_training_environment()

    def run_benchmark(self, size_spec: str) -> None:
        """Like :meth:`run` with no checkpoints, no evaluation, the profiler on and a hard stop after 100 steps."""
        self.run(size_spec, for_benchmarking=True)

    # -- inspecting results ------------------------------------------------------------------------------------
    def get_checkpoints(self, size_spec: str, download_metrics: bool = False, discover_all: bool = False,
                        alternative_dirs: Optional[List[PathOrStr]] = None) -> List[RunCheckpointInfo]:
        """
        The rung's checkpoints in step order: by default the planned ones (present or not), with ``discover_all`` whatever
        exists on disk. Each step is looked up in the save folder first, then in ``<alt>/<size>`` for every alternative.
        """
        primary = self.get_save_folder(size_spec)
        folders = [primary] + [str(io.join_path(d, size_spec)) for d in (alternative_dirs or [])]
        for folder in folders:
            io.init_client(folder)
        n = self.get_num_params(size_spec)
        batch = self._configure_batch_size_and_num_devices(size_spec, n)[0]

        wanted: Dict[int, Tuple[str, Optional[PathOrStr]]] = {}
        if discover_all:
            for folder in folders:
                try:
                    for step, path in Checkpointer.find_checkpoints(folder):
                        wanted.setdefault(step, (f"step-{step}", path))
                except FileNotFoundError:
                    pass
        else:
            wanted[0] = ("initialization", None)
            plan = self.run_configurator.configure_checkpoint_intervals(n, batch)
            for step, (_, label) in zip(self._get_checkpoint_intervals(num_params=n, global_batch_size=batch), plan):
                wanted[step] = (label, None)

        def describe(step: int, label: str, path: Optional[PathOrStr]) -> RunCheckpointInfo:
            exists = False
            if path is not None:
                exists = Checkpointer.dir_is_checkpoint(path)
            else:
                name = Checkpointer.checkpoint_dirname(step)
                path = io.join_path(primary, name)
                for folder in folders:
                    candidate = io.join_path(folder, name)
                    if Checkpointer.dir_is_checkpoint(candidate):
                        path, exists = candidate, True
                        break
            metrics: Optional[PathOrStr] = None
            for folder in folders:
                candidate = io.join_path(folder, f"metrics_step{step}.json")
                if io.file_exists(candidate):
                    metrics = candidate
                    break
            if metrics is not None and download_metrics and io.is_url(metrics):
                local = io.join_path(self.work_dir, f"{size_spec}-metrics_step{step}.json")
                io.copy_file(metrics, local, save_overwrite=True)
                metrics = local
            return RunCheckpointInfo(name=label, step=step, tokens=step * batch, path=path, metrics_path=metrics,
                                     exists=exists)

        with concurrent.futures.ThreadPoolExecutor() as pool:
            infos = list(pool.map(lambda item: describe(item[0], item[1][0], item[1][1]), wanted.items()))
        return sorted(infos, key=lambda info: info.step)

    def get_metrics(self, size_spec: str, prefix: Optional[str] = None, discover_all: bool = False,
                    alternative_dirs: Optional[List[PathOrStr]] = None):
        """One row per checkpoint that has a metrics file (a ``pandas.DataFrame``), or ``None``."""
        import pandas as pd

        n = self.get_num_params(size_spec)
        rows = []
        for ckpt in self.get_checkpoints(size_spec, download_metrics=True, discover_all=discover_all,
                                         alternative_dirs=alternative_dirs):
            if ckpt.metrics_path is None:
                continue
            with open(ckpt.metrics_path) as f:
                metrics = json.load(f)
            if prefix is not None:
                metrics = {k: v for k, v in metrics.items() if k.startswith(prefix)}
            metrics.update(name=ckpt.name, step=ckpt.step, tokens=ckpt.tokens, size=size_spec, num_params=n)
            rows.append(metrics)
        return pd.DataFrame(rows) if rows else None
