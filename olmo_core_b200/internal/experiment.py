"""
Sub-command CLI shared by experiment scripts (role of src/olmo_core/internal/experiment.py:56-535)::

    python script.py {launch|train|train_single|prep|launch_prep|dry_run} RUN_NAME CLUSTER [key=value overrides ...]

A script passes a ``config_builder(CliContext) -> ExperimentConfig``; :func:`build_config` assembles one from small
per-component builders with sensible defaults. ``CLUSTER`` may be ``local`` for a run on this machine's GPUs.
"""

from __future__ import annotations

import logging
import sys
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Union, cast

import torch

from ..config import Config, StrEnum
from ..data import (
    DataLoaderBase,
    DataMix,
    InstanceFilterConfig,
    NumpyDataLoaderConfig,
    NumpyDatasetConfig,
    NumpyFSLDatasetConfig,
    NumpyPaddedFSLDatasetConfig,
    TokenizerConfig,
)
from ..distributed.utils import get_local_rank
from ..launch.beaker import BeakerLaunchConfig, OLMoCoreBeakerImage
from ..nn.transformer import TransformerConfig
from ..train import TrainerConfig, prepare_training_environment, teardown_training_environment
from ..train.callbacks import (
    BeakerCallback,
    Callback,
    ConfigSaverCallback,
    DownstreamEvaluatorCallbackConfig,
    GAPMonitorCallback,
    GarbageCollectorCallback,
    GPUMemoryMonitorCallback,
    LMEvaluatorCallbackConfig,
    ProfilerCallback,
    SlackNotifierCallback,
)
from ..train.train_module import TransformerTrainModuleConfig
from ..utils import prepare_cli_environment, seed_all
from .common import build_launch_config, get_beaker_username, get_root_dir, get_work_dir

log = logging.getLogger(__name__)

__all__ = ["CliContext", "CommonComponents", "DataComponents", "ExperimentConfig", "SubCmd", "ConfigBuilder",
           "build_common_components", "build_default_data_components", "build_config", "launch", "launch_prep", "prep",
           "train", "main"]


class SubCmd(StrEnum):
    launch = "launch"
    train = "train"
    train_single = "train_single"
    prep = "prep"
    launch_prep = "launch_prep"
    dry_run = "dry_run"

    def post_launch_subcmd(self) -> "SubCmd":
        """What the launched job itself runs."""
        return SubCmd.prep if self in (SubCmd.prep, SubCmd.launch_prep) else SubCmd.train

    def prepare_environment(self, config: "ExperimentConfig") -> None:
        if self == SubCmd.train:
            prepare_training_environment(backend=config.backend)
        elif self == SubCmd.train_single:
            prepare_training_environment(backend=None)
        else:
            prepare_cli_environment()

    def run(self, config: "ExperimentConfig") -> None:
        if get_local_rank() == 0:
            print(config)
            m = config.model
            print(f"\nTotal parameters:         {m.num_params:,d} ({m.num_active_params:,d} active)\n"
                  f"Non-embedding parameters: {m.num_non_embedding_params:,d} "
                  f"({m.num_active_non_embedding_params:,d} active)")
        if self == SubCmd.dry_run:
            return
        if self == SubCmd.launch:
            launch(config)
        elif self == SubCmd.launch_prep:
            launch_prep(config)
        elif self == SubCmd.prep:
            prep(config)
        else:
            if self == SubCmd.train_single:
                for name in ("dp_config", "tp_config"):
                    if getattr(config.train_module, name, None) is not None:
                        log.warning("'%s' is set but a single-device run cannot use it; disabling", name)
                        setattr(config.train_module, name, None)
            train(config)
            teardown_training_environment()


@dataclass
class CliContext(Config):
    script: str
    cmd: SubCmd
    run_name: str
    cluster: str
    overrides: List[str]

    @property
    def remote_cmd(self) -> List[str]:
        return [self.script, str(self.cmd.post_launch_subcmd()), self.run_name, self.cluster, *self.overrides]


@dataclass
class CommonComponents(Config):
    run_name: str
    root_dir: str
    work_dir: str
    save_folder: str
    launch: Optional[BeakerLaunchConfig]
    tokenizer: TokenizerConfig
    max_sequence_length: int
    global_batch_size: int


@dataclass
class DataComponents(Config):
    dataset: Union[NumpyDatasetConfig, List[Any]]
    data_loader: Any


@dataclass
class ExperimentConfig(Config):
    run_name: str
    launch: Optional[BeakerLaunchConfig]
    model: TransformerConfig
    dataset: Union[NumpyDatasetConfig, List[Any]]
    data_loader: Any
    train_module: Any
    trainer: TrainerConfig
    init_seed: int = 12536
    backend: Optional[str] = "cpu:gloo,cuda:nccl"


ConfigBuilder = Callable[[CliContext], ExperimentConfig]


def build_common_components(cli_context: CliContext, *, tokenizer: TokenizerConfig, global_batch_size: int,
                            max_sequence_length: int, beaker_image: str = OLMoCoreBeakerImage.stable, num_nodes: int = 1,
                            beaker_workspace: str = "ai2/OLMo-core", num_execution_units: Optional[int] = None,
                            flight_recorder: bool = False) -> CommonComponents:
    root_dir = get_root_dir(cli_context.cluster)
    user = get_beaker_username()
    launch_config = None
    if user is not None:
        job = cli_context.cmd.post_launch_subcmd()
        launch_config = build_launch_config(
            name=f"{cli_context.run_name}-{job}", root_dir=root_dir, cmd=cli_context.remote_cmd,
            cluster=cli_context.cluster, nccl_debug=True, flight_recorder=flight_recorder, beaker_image=beaker_image,
            num_nodes=num_nodes, workspace=beaker_workspace, num_execution_units=num_execution_units)
        launch_config.launch_timeout = 5 * 60
    owner = f"{user.lower()}/" if user is not None else ""
    return CommonComponents(
        run_name=cli_context.run_name, root_dir=root_dir, work_dir=get_work_dir(root_dir),
        save_folder=f"{root_dir}/checkpoints/{owner}{cli_context.run_name}", launch=launch_config, tokenizer=tokenizer,
        max_sequence_length=max_sequence_length, global_batch_size=global_batch_size)


def build_default_data_components(common: CommonComponents, intra_document_masking: bool = False,
                                  include_instance_filter: bool = False) -> DataComponents:
    """A fixed-sequence-length dataset over the default pre-training mix plus a matching loader."""
    dataset = NumpyFSLDatasetConfig.from_data_mix(
        DataMix.OLMoE_mix_0824, tokenizer=common.tokenizer, mix_base_dir=common.root_dir, work_dir=common.work_dir,
        sequence_length=common.max_sequence_length, max_target_sequence_length=max(common.max_sequence_length, 8192),
        generate_doc_lengths=intra_document_masking,
        instance_filter_config=(InstanceFilterConfig(repetition_max_period=13, repetition_min_period=1,
                                                     repetition_max_count=32) if include_instance_filter else None))
    loader = NumpyDataLoaderConfig(global_batch_size=common.global_batch_size, seed=34521, num_workers=4)
    return DataComponents(dataset=dataset, data_loader=loader)


def _required_callbacks(common: CommonComponents) -> Dict[str, Callback]:
    callbacks: Dict[str, Callback] = {
        "config_saver": ConfigSaverCallback(),
        "profiler": ProfilerCallback(enabled=False),
        "garbage_collector": GarbageCollectorCallback(),
        "slack_notifier": SlackNotifierCallback(name=common.run_name, enabled=False),
        "gap_monitor": GAPMonitorCallback(enabled=False),
    }
    if common.launch is not None:
        callbacks["beaker"] = BeakerCallback()
    if torch.cuda.is_available():
        callbacks["gpu_monitor"] = GPUMemoryMonitorCallback()
    return callbacks


def _default_eval_callbacks(common: CommonComponents) -> Dict[str, Any]:
    return {
        "lm_evaluator": LMEvaluatorCallbackConfig(
            eval_dataset=NumpyPaddedFSLDatasetConfig.from_data_mix(
                DataMix.v3_small_ppl_validation, mix_base_dir=common.root_dir,
                sequence_length=common.max_sequence_length, tokenizer=common.tokenizer, work_dir=common.work_dir),
            eval_interval=1000),
        "downstream_evaluator": DownstreamEvaluatorCallbackConfig(tasks=["hellaswag"], tokenizer=common.tokenizer,
                                                                  eval_interval=1000),
    }


def build_config(cli_context: CliContext, *, model_config_builder: Callable[[CommonComponents], TransformerConfig],
                 train_module_config_builder: Callable[[CommonComponents], TransformerTrainModuleConfig],
                 trainer_config_builder: Callable[[CommonComponents], TrainerConfig], global_batch_size: int,
                 common_config_builder: Callable[..., CommonComponents] = build_common_components,
                 data_config_builder: Callable[..., DataComponents] = build_default_data_components,
                 finalize_config: Optional[Callable[[ExperimentConfig], None]] = None,
                 tokenizer: Optional[TokenizerConfig] = None, max_sequence_length: int = 4096,
                 beaker_image: str = OLMoCoreBeakerImage.stable, num_nodes: int = 1,
                 beaker_workspace: str = "ai2/OLMo-core", flight_recorder: bool = False,
                 num_execution_units: Optional[int] = None, include_default_evals: bool = False,
                 **data_kwargs) -> ExperimentConfig:
    """
    Assemble an :class:`ExperimentConfig`: common components first, then data / model / trainer / train module from their
    builders; required callbacks (and optionally default evaluators) are added unless the trainer config already has a
    callback under that name; command-line overrides are merged last, then ``finalize_config`` may edit in place.
    """
    common = common_config_builder(
        cli_context, tokenizer=tokenizer or TokenizerConfig.dolma2(), global_batch_size=global_batch_size,
        max_sequence_length=max_sequence_length, beaker_image=beaker_image, num_nodes=num_nodes,
        beaker_workspace=beaker_workspace, flight_recorder=flight_recorder, num_execution_units=num_execution_units)
    data = data_config_builder(common, **data_kwargs)
    model = model_config_builder(common)
    trainer = trainer_config_builder(common)
    extra: Dict[str, Any] = _required_callbacks(common)
    if include_default_evals:
        extra.update(_default_eval_callbacks(common))
    for name, callback in extra.items():
        if name not in trainer.callbacks:
            trainer.add_callback(name, callback)
    config = ExperimentConfig(run_name=cli_context.run_name, launch=common.launch, model=model, dataset=data.dataset,
                              data_loader=data.data_loader, train_module=train_module_config_builder(common),
                              trainer=trainer)
    config = config.merge(cli_context.overrides)
    if finalize_config is not None:
        finalize_config(config)
    return config


def launch(config: ExperimentConfig) -> None:
    if config.launch is None:
        raise RuntimeError("no launch configuration: Beaker is not configured in this environment")
    config.launch.launch()


def launch_prep(config: ExperimentConfig) -> None:
    if config.launch is None:
        raise RuntimeError("no launch configuration: Beaker is not configured in this environment")
    config.launch.num_gpus, config.launch.num_nodes = 0, 1
    config.launch.launch(torchrun=False)


def _build_data_loader(config: ExperimentConfig, dp_process_group=None) -> DataLoaderBase:
    if isinstance(config.data_loader, NumpyDataLoaderConfig):
        assert isinstance(config.dataset, NumpyDatasetConfig)
        return config.data_loader.build(config.dataset.build(), dp_process_group=dp_process_group)
    if isinstance(config.dataset, list):  # composable sources
        work_dir = getattr(config.data_loader, "work_dir", None)
        if work_dir is None:
            raise ValueError("Please set 'work_dir' on the data loader config")
        sources = [source.build(work_dir) for source in config.dataset]
        return config.data_loader.build(*sources, dp_process_group=dp_process_group)
    raise NotImplementedError(type(config.data_loader))


def prep(config: ExperimentConfig) -> None:
    """Do the dataset preprocessing (index files, global shuffle order) ahead of the GPU job."""
    _build_data_loader(config).reshuffle(epoch=1)


def train(config: ExperimentConfig) -> None:
    seed_all(config.init_seed)
    model = config.model.build(init_device="meta")
    train_module = config.train_module.build(model)
    data_loader = _build_data_loader(config, dp_process_group=train_module.dp_process_group)
    trainer = config.trainer.build(train_module, data_loader)
    cast(ConfigSaverCallback, trainer.callbacks["config_saver"]).config = config.as_config_dict()
    trainer.fit()


def _usage() -> str:
    s = sys.argv[0]
    return (f"Usage: python {s} {'|'.join(SubCmd)} RUN_NAME CLUSTER [OVERRIDES...]\n\n"
            "  launch        submit the script to Beaker with the 'train' sub-command\n"
            "  train         run the trainer (start it with torchrun, or through 'launch')\n"
            "  train_single  run the trainer on one device, parallelism disabled\n"
            "  prep          prepare the dataset ahead of training\n"
            "  launch_prep   submit the script to Beaker with the 'prep' sub-command\n"
            "  dry_run       print the config and exit\n\n"
            f"Example: python {s} {SubCmd.launch} run01 ai2/jupiter --launch.num_nodes=2")


def main(*, config_builder: ConfigBuilder) -> None:
    if len(sys.argv) < 4 or sys.argv[1] not in set(SubCmd):
        print(_usage())
        sys.exit(1)
    script, cmd_name, run_name, cluster, *overrides = sys.argv
    cmd = SubCmd(cmd_name)
    config = config_builder(CliContext(script, cmd, run_name, cluster, overrides))
    cmd.prepare_environment(config)
    cmd.run(config)
