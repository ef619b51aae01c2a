"""
Ready-made pieces of an experiment config (role of src/olmo_core/internal/cookbook.py:44-156): the usual train-module
settings (SkipStepAdamW, HSDP in bf16 with fp32 reduction, z-loss, gradient clipping at 1.0), a trainer config with the
load strategy derived from ``load_path``, and the standard callback sets.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config import DType
from ..distributed.parallel import DataParallelType
from ..float8 import AOFloat8LinearConfig, Float8Config
from ..io import dir_is_empty
from ..optim import OptimGroupOverride, Scheduler, SkipStepAdamWConfig
from ..train import Duration, LoadStrategy, TrainerConfig
from ..train.callbacks import (
    BeakerCallback,
    Callback,
    CheckpointerCallback,
    ConfigSaverCallback,
    GAPMonitorCallback,
    GarbageCollectorCallback,
    GPUMemoryMonitorCallback,
    ProfilerCallback,
    SlackNotifierCallback,
    WandBCallback,
)
from ..train.train_module import (
    TransformerActivationCheckpointingConfig,
    TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig,
    TransformerDataParallelConfig,
    TransformerTrainModuleConfig,
)
from .common import get_beaker_username

__all__ = ["configure_train_module", "configure_trainer", "configure_required_callbacks", "configure_default_callbacks"]


def configure_train_module(max_sequence_length: int, rank_microbatch_size: int, learning_rate: float, scheduler: Scheduler,
                           float8_enabled: bool = False, activation_memory_budget: float = 1.0,
                           dp_shard_degree: Optional[int] = None, cp_degree: Optional[int] = None
                           ) -> TransformerTrainModuleConfig:
    """``activation_memory_budget`` below 1.0 turns on budget-mode activation checkpointing (smaller = more recompute)."""
    if not 0.0 < activation_memory_budget <= 1.0:
        raise ValueError("activation_memory_budget must be in the range (0.0, 1.0].")
    ac = None
    if activation_memory_budget < 1.0:
        ac = TransformerActivationCheckpointingConfig(mode=TransformerActivationCheckpointingMode.budget,
                                                      activation_memory_budget=activation_memory_budget)
    return TransformerTrainModuleConfig(
        rank_microbatch_size=rank_microbatch_size, max_sequence_length=max_sequence_length,
        optim=SkipStepAdamWConfig(lr=learning_rate, weight_decay=0.1, betas=(0.9, 0.95), foreach=True,
                                  group_overrides=[OptimGroupOverride(params=["embeddings.weight"],
                                                                      opts=dict(weight_decay=0.0))]),
        scheduler=scheduler, z_loss_multiplier=1e-5, max_grad_norm=1.0, compile_model=True,
        dp_config=TransformerDataParallelConfig(name=DataParallelType.hsdp, param_dtype=DType.bfloat16,
                                                reduce_dtype=DType.float32, shard_degree=dp_shard_degree),
        cp_config=TransformerContextParallelConfig.llama3(degree=cp_degree, head_stride=4) if cp_degree else None,
        ac_config=ac, float8_config=Float8Config(enabled=float8_enabled, ao=AOFloat8LinearConfig.recommended()))


def configure_trainer(max_duration: Duration, checkpoint_dir: str, work_dir: str, load_path: Optional[str] = None,
                      load_trainer_state: Optional[bool] = None, load_optim_state: Optional[bool] = None,
                      hard_stop: Optional[Duration] = None) -> TrainerConfig:
    if load_path and dir_is_empty(load_path):
        raise FileNotFoundError(f"load_path={load_path!r} was provided, but the directory is empty.")
    return TrainerConfig(max_duration=max_duration, load_path=load_path, save_folder=checkpoint_dir, work_dir=work_dir,
                         hard_stop=hard_stop, load_strategy=LoadStrategy.always if load_path else LoadStrategy.if_available,
                         load_trainer_state=load_trainer_state, load_optim_state=load_optim_state, save_overwrite=True)


def configure_required_callbacks(run_name: str) -> Dict[str, Callback]:
    callbacks: Dict[str, Callback] = {
        "config_saver": ConfigSaverCallback(),
        "profiler": ProfilerCallback(enabled=False),
        "garbage_collector": GarbageCollectorCallback(),
        "slack_notifier": SlackNotifierCallback(name=run_name, enabled=False),
        "gap_monitor": GAPMonitorCallback(enabled=False),
    }
    if get_beaker_username() is not None:
        callbacks["beaker"] = BeakerCallback()
    if torch.cuda.is_available():
        callbacks["gpu_monitor"] = GPUMemoryMonitorCallback()
    return callbacks


def configure_default_callbacks(run_name: str, wandb_group_name: str, wandb_project: str = "olmo-cookbook",
                                checkpoint_save_interval: Optional[int] = 1000,
                                ephemeral_checkpoint_save_interval: Optional[int] = None) -> Dict[str, Callback]:
    callbacks = configure_required_callbacks(run_name)
    callbacks["checkpointer"] = CheckpointerCallback(save_interval=checkpoint_save_interval,
                                                     ephemeral_save_interval=ephemeral_checkpoint_save_interval,
                                                     save_async=True)
    callbacks["wandb"] = WandBCallback(name=run_name, group=wandb_group_name, project=wandb_project, entity="ai2-llm",
                                       cancel_check_interval=20, enabled=True)
    return callbacks
