"""
Training loop, train modules, callbacks and checkpointing
(public names of src/olmo_core/train/__init__.py:43-160).

Typical script::

    prepare_training_environment(seed=0)
    try:
        trainer = trainer_config.build(train_module, data_loader)
        trainer.fit()
    finally:
        teardown_training_environment()
"""

import logging
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ..distributed.utils import init_distributed, is_distributed
from ..io import add_cached_path_clients
from ..utils import LogFilterType, get_default_device, prepare_cli_environment, seed_all
from .checkpoint import Checkpointer, CheckpointerConfig
from .common import Duration, DurationUnit, LoadStrategy, MetricMergeStrategy, ReduceType, StepSkipRange
from .config import TrainerConfig
from .trainer import Trainer

__all__ = [
    "prepare_training_environment",
    "teardown_training_environment",
    "TrainerConfig",
    "Trainer",
    "CheckpointerConfig",
    "Checkpointer",
    "LoadStrategy",
    "Duration",
    "DurationUnit",
    "ReduceType",
    "MetricMergeStrategy",
    "StepSkipRange",
]

log = logging.getLogger(__name__)


def prepare_training_environment(*, seed: Optional[int] = None, backend: Optional[str] = "cpu:gloo,cuda:nccl",
                                 timeout: timedelta = timedelta(minutes=15),
                                 log_filter_type: Optional[LogFilterType] = None,
                                 shared_filesystem: Optional[bool] = None) -> None:
    """
    Call first in a training script: initialises the process group (one process per GPU; NCCL for device tensors
    plus gloo so that checkpointing and bookkeeping collectives run on the host, off the training stream), binds
    the process to its GPU, configures logging / exception hooks and seeds the RNGs. ``backend=None`` runs
    single-process.
    """
    try:
        mp.set_start_method("spawn", force=True)  # data-loader workers must not inherit a CUDA context by fork
    except RuntimeError as e:
        print(f"failed to set multiprocessing start method: {e}")
    if backend is not None:
        init_distributed(backend=backend, timeout=timeout, shared_filesystem=shared_filesystem)
    else:
        torch.set_default_device(get_default_device())
    prepare_cli_environment(log_filter_type=log_filter_type)
    add_cached_path_clients()
    if seed is not None:
        seed_all(seed)
    if is_distributed():
        log.info(f"Using distributed backend {dist.get_backend()}")


def teardown_training_environment() -> None:
    """Call last: destroys all process groups."""
    if is_distributed():
        dist.destroy_process_group()
