"""
The :class:`TrainModule` interface between the :class:`~olmo_core_b200.train.Trainer` and a model +
optimizer, and a basic single-model implementation (src/olmo_core/train/train_module/train_module.py:27-413).
"""

from __future__ import annotations

from abc import ABCMeta, abstractmethod
from dataclasses import dataclass
from typing import TYPE_CHECKING, Any, Dict, Optional, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ...config import StrEnum
from ...data.utils import get_labels, split_batch
from ...exceptions import OLMoConfigurationError
from ...optim import OptimConfig, SkipStepOptimizer
from ...optim.scheduler import Scheduler
from ...utils import get_default_device, move_to_device
from ..common import MetricMergeStrategy, ReduceType

if TYPE_CHECKING:
    from ..trainer import Trainer

__all__ = ["TrainModule", "EvalBatchSpec", "EvalBatchSizeUnit", "BasicTrainModule"]


class EvalBatchSizeUnit(StrEnum):
    tokens = "tokens"
    instances = "instances"


@dataclass
class EvalBatchSpec:
    rank_batch_size: int
    batch_size_unit: EvalBatchSizeUnit = EvalBatchSizeUnit.tokens
    max_sequence_length: Optional[int] = None
    fixed_sequence_length: bool = False

    def __post_init__(self):
        if self.fixed_sequence_length and self.max_sequence_length is None:
            raise OLMoConfigurationError("'max_sequence_length' must be specified when 'fixed_sequence_length=True'")


class TrainModule(metaclass=ABCMeta):
    """Owns the model and optimizer; the trainer calls it once per batch."""

    def __init__(self):
        self._trainer: Optional["Trainer"] = None

    @property
    def trainer(self) -> "Trainer":
        if self._trainer is None:
            raise RuntimeError("trainer has not been attached yet")
        return self._trainer

    @property
    def dp_process_group(self) -> Optional[dist.ProcessGroup]:
        return None

    @property
    @abstractmethod
    def eval_batch_spec(self) -> EvalBatchSpec:
        raise NotImplementedError

    def on_attach(self) -> None:
        """Called once the trainer is available (validate batch sizes here)."""

    def pre_train(self) -> None:
        """Called right before the first step."""

    @abstractmethod
    def state_dict(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        raise NotImplementedError

    def state_dict_to_save(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        return self.state_dict(optim=optim)

    def state_dict_to_load(self, metadata, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        del metadata
        return self.state_dict(optim=optim)

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        raise NotImplementedError

    @abstractmethod
    def train_batch(self, batch: Dict[str, Any], dry_run: bool = False):
        raise NotImplementedError

    @abstractmethod
    def eval_batch(self, batch: Dict[str, Any], labels: Optional[Any] = None) -> Any:
        raise NotImplementedError

    @abstractmethod
    def optim_step(self):
        raise NotImplementedError

    @abstractmethod
    def zero_grads(self):
        raise NotImplementedError

    @abstractmethod
    def num_flops_per_token(self, seq_len: int) -> Optional[int]:
        raise NotImplementedError

    @abstractmethod
    def global_num_flops_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        raise NotImplementedError

    def record_metric(self, name: str, value: Union[float, torch.Tensor], reduce_type: Optional[ReduceType] = None,
                      namespace: Optional[str] = None, merge_strategy: MetricMergeStrategy = MetricMergeStrategy.warn) -> None:
        if self._trainer is not None:
            self._trainer.record_metric(name, value, reduce_type=reduce_type, namespace=namespace, merge_strategy=merge_strategy)

    def record_ce_loss(self, value: Union[float, torch.Tensor], reduce_type: Optional[ReduceType] = None) -> None:
        if self._trainer is not None:
            self._trainer.record_ce_loss(value, reduce_type=reduce_type)

    def _attach_trainer(self, trainer: "Trainer") -> None:
        self._trainer = trainer
        self.on_attach()


class BasicTrainModule(TrainModule):
    """
    Train module for any ``nn.Module`` with a loss function ``loss_fn(output, labels) -> scalar`` (summed over
    tokens): micro-batching, gradient accumulation, optional clipping and scheduler.
    """

    def __init__(self, model: nn.Module, optim: OptimConfig, rank_microbatch_size: int, loss_fn=None,
                 max_grad_norm: Optional[float] = None, scheduler: Optional[Scheduler] = None,
                 device: Optional[torch.device] = None, label_ignore_index: int = -100):
        super().__init__()
        self.device = device or get_default_device()
        self.model = model.to(self.device)
        self.optim = optim.build(self.model)
        self.rank_microbatch_size = rank_microbatch_size
        self.max_grad_norm = max_grad_norm
        self.scheduler = scheduler
        self.label_ignore_index = label_ignore_index
        self.loss_fn = loss_fn or (lambda logits, labels: torch.nn.functional.cross_entropy(
            logits.float().view(-1, logits.size(-1)), labels.view(-1), ignore_index=label_ignore_index, reduction="sum"))

    @property
    def eval_batch_spec(self) -> EvalBatchSpec:
        return EvalBatchSpec(rank_batch_size=self.rank_microbatch_size)

    def on_attach(self) -> None:
        rbz = self.trainer.rank_batch_size
        if rbz % self.rank_microbatch_size != 0:
            raise OLMoConfigurationError(f"rank batch size ({rbz}) must be divisible by the micro-batch size ({self.rank_microbatch_size})")

    def state_dict(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        sd: Dict[str, Any] = {"model": self.model.state_dict()}
        if optim is not False:
            sd["optim"] = self.optim.state_dict()
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self.model.load_state_dict(state_dict["model"])
        if "optim" in state_dict:
            self.optim.load_state_dict(state_dict["optim"])

    def model_forward(self, micro_batch: Dict[str, Any]) -> torch.Tensor:
        return self.model(micro_batch["input_ids"])

    def train_batch(self, batch: Dict[str, Any], dry_run: bool = False):
        self.model.train()
        if "labels" not in batch:
            batch["labels"] = get_labels(batch, self.label_ignore_index)
        n_tokens = (batch["labels"] != self.label_ignore_index).sum().clamp(min=1)
        seq_len = batch["input_ids"].shape[1]
        total = torch.zeros((), device=self.device)
        for mb in split_batch(batch, max(1, self.rank_microbatch_size // seq_len)):
            mb = move_to_device(mb, self.device)
            loss = self.loss_fn(self.model_forward(mb), mb["labels"]) / n_tokens.to(self.device)
            total += loss.detach()
            loss.backward()
        if not dry_run:
            self.record_ce_loss(total, ReduceType.mean)

    def eval_batch(self, batch: Dict[str, Any], labels: Optional[torch.Tensor] = None) -> Any:
        self.model.eval()
        batch = move_to_device(batch, self.device)
        with torch.no_grad():
            logits = self.model_forward(batch)
        if labels is None:
            return logits
        return logits, self.loss_fn(logits, move_to_device(labels, self.device))

    def optim_step(self):
        if self.max_grad_norm is not None:
            norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
            self.record_metric("total grad norm", norm, reduce_type=None, namespace="optim")
            if isinstance(self.optim, SkipStepOptimizer):
                self.optim.latest_grad_norm = norm
        if self.scheduler is not None:
            for i, group in enumerate(self.optim.param_groups):
                lr = self.scheduler.set_lr(group, self.trainer)
                self.record_metric(f"LR (group {i})", lr, namespace="optim")
        self.optim.step()

    def zero_grads(self):
        self.optim.zero_grad(set_to_none=True)

    def num_flops_per_token(self, seq_len: int) -> Optional[int]:
        fn = getattr(self.model, "num_flops_per_token", None)
        return fn(seq_len) if fn is not None else None

    def global_num_flops_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        per_tok = self.num_flops_per_token(batch["input_ids"].shape[1])
        return None if per_tok is None else per_tok * self.trainer.data_loader.global_num_tokens_in_batch(batch)
