"""Serialisable trainer settings (fields and ``build`` of src/olmo_core/train/config.py:22-230)."""

from __future__ import annotations

import os
import tempfile
from copy import deepcopy
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..config import Config
from ..exceptions import OLMoConfigurationError
from ..io import is_url
from ..utils import get_default_device
from .callbacks import Callback, CallbackConfig
from .checkpoint import CheckpointerConfig
from .common import Duration, LoadStrategy, StepSkipRange
from .train_module import TrainModule
from .trainer import Trainer

__all__ = ["TrainerConfig"]


@dataclass
class TrainerConfig(Config):
    """See :class:`Trainer` for the meaning of the fields."""

    save_folder: str
    work_dir: Optional[str] = None
    load_path: Optional[str] = None
    load_strategy: LoadStrategy = LoadStrategy.if_available
    load_optim_state: Optional[bool] = None
    load_trainer_state: Optional[bool] = None
    checkpointer: CheckpointerConfig = field(default_factory=CheckpointerConfig)
    device: Optional[str] = None
    save_overwrite: bool = False
    max_duration: Duration = field(default_factory=lambda: Duration.epochs(1))
    cancel_check_interval: int = 25
    hard_stop: Optional[Duration] = None
    metrics_collect_interval: int = 5
    callbacks: Dict[str, Callback] = field(default_factory=dict)
    async_bookkeeping: Optional[bool] = None
    bookkeeping_soft_timeout: int = 30
    no_checkpoints: bool = False
    no_evals: bool = False
    steps_to_skip: Optional[List[StepSkipRange]] = None

    def add_callback(self, name: str, callback: Callback) -> None:
        if name in self.callbacks:
            raise OLMoConfigurationError(f"A callback with name '{name}' already exists")
        self.callbacks[name] = callback

    def add_callbacks(self, callbacks: Dict[str, Callback]) -> None:
        for name, cb in callbacks.items():
            self.add_callback(name, cb)

    def with_callback(self, name: str, callback: Callback) -> "TrainerConfig":
        """A copy of this config with one more callback."""
        return self.with_callbacks({name: callback})

    def with_callbacks(self, callbacks: Dict[str, Callback]) -> "TrainerConfig":
        out = replace(self, callbacks=deepcopy(self.callbacks))
        out.add_callbacks(callbacks)
        return out

    def with_recommended_evals(self, tokenizer, sequence_length: int, cluster: str, task_set: str = "full",
                               eval_interval: int = 10_000, lazy_load: bool = False) -> "TrainerConfig":
        """Adds the downstream task suite ``task_set`` and perplexity over the small validation mix."""
        from ..data import DataMix, NumpyPaddedFSLDatasetConfig
        from ..eval.task_groups import TASK_GROUPS
        from ..internal.common import get_root_dir, get_work_dir
        from .callbacks import DownstreamEvaluatorCallbackConfig, LMEvaluatorCallbackConfig

        if task_set not in TASK_GROUPS:
            raise ValueError(f"Task set not recognized: {task_set}")
        root = get_root_dir(cluster)
        return self.with_callbacks({
            "downstream_evaluator": DownstreamEvaluatorCallbackConfig(
                tasks=sorted(TASK_GROUPS[task_set]), tokenizer=tokenizer, eval_interval=eval_interval, lazy=lazy_load,
                eval_on_finish=True),
            "lm_evaluator": LMEvaluatorCallbackConfig(
                eval_dataset=NumpyPaddedFSLDatasetConfig.from_data_mix(
                    DataMix.v3_small_ppl_validation, mix_base_dir=root, sequence_length=sequence_length,
                    tokenizer=tokenizer, work_dir=get_work_dir(root)),
                eval_interval=eval_interval, eval_on_finish=True),
        })

    def build(self, train_module: TrainModule, data_loader: Any, *, dp_process_group: Optional[dist.ProcessGroup] = None,
              checkpointer_pg: Optional[dist.ProcessGroup] = None) -> Trainer:
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        device = kwargs.pop("device", None)
        work_dir = kwargs.pop("work_dir", None)
        if work_dir is None:
            # a local save folder doubles as scratch space; a remote one gets a temp dir named after it
            work_dir = self.save_folder if not is_url(self.save_folder) else os.path.join(
                tempfile.gettempdir(), os.path.basename(self.save_folder.rstrip("/")))
        elif is_url(work_dir):
            raise OLMoConfigurationError(f"Trainer 'work_dir' must be a local path, not a URL ('{work_dir}')")
        ckpt_kwargs: Dict[str, Any] = {}
        if self.checkpointer.save_overwrite is None:
            ckpt_kwargs["save_overwrite"] = self.save_overwrite
        if self.checkpointer.work_dir is None:
            ckpt_kwargs["work_dir"] = work_dir
        checkpointer = kwargs.pop("checkpointer").build(process_group=checkpointer_pg, **ckpt_kwargs)
        every = kwargs.pop("callbacks")
        ready = {k: cb for k, cb in every.items() if not isinstance(cb, CallbackConfig)}
        deferred = {k: cb for k, cb in every.items() if isinstance(cb, CallbackConfig)}
        trainer = Trainer(
            train_module=train_module, data_loader=data_loader, checkpointer=checkpointer, work_dir=Path(work_dir),
            device=torch.device(device) if device is not None else get_default_device(),
            dp_process_group=dp_process_group if dp_process_group is not None else train_module.dp_process_group,
            callbacks=ready, **kwargs,
        )
        for name, cfg in deferred.items():  # these need the finished trainer (data loader, batch spec, ...)
            cb = cfg.build(trainer)
            if cb is not None:
                trainer.add_callback(name, cb)
        return trainer
