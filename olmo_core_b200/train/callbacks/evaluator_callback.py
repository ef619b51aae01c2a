"""
In-loop evaluation (options and metric names of src/olmo_core/train/callbacks/evaluator_callback.py:45-524).

:class:`EvaluatorCallback` runs a list of :class:`~olmo_core_b200.eval.Evaluator` every ``eval_interval`` steps (and at
``fixed_steps``, on start-up, at the end) through the train module's ``eval_batch`` and records
``eval/<evaluator>/<metric>``. Two config front-ends build it: perplexity over labelled validation sets
(:class:`LMEvaluatorCallbackConfig`) and the ``olmo_eval`` in-context-learning task suite
(:class:`DownstreamEvaluatorCallbackConfig`; needs the optional ``olmo_eval`` package).
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from functools import lru_cache
from typing import TYPE_CHECKING, Any, Dict, List, Optional, Set

import torch
import torch.distributed as dist

from ...data.utils import get_labels
from ...distributed.utils import get_rank, get_world_size, is_distributed
from ...eval import Evaluator, LMEvaluator
from ...exceptions import OLMoConfigurationError
from ...utils import cuda_sync_debug_mode, format_float, gc_cuda, get_default_device, move_to_device
from ..common import Duration, MetricMergeStrategy
from ..train_module import EvalBatchSizeUnit, EvalBatchSpec
from .callback import Callback, CallbackConfig

if TYPE_CHECKING:
    from ..trainer import Trainer

log = logging.getLogger(__name__)

__all__ = ["EvaluatorCallback", "LMEvaluatorCallbackConfig", "DownstreamEvaluator", "DownstreamEvaluatorCallbackConfig"]


@dataclass
class EvaluatorCallback(Callback):
    evaluators: List[Evaluator] = field(default_factory=list)
    eval_interval: Optional[int] = 1000
    fixed_steps: Optional[List[int]] = None
    eval_on_startup: bool = False
    eval_on_finish: bool = False
    cancel_after_first_eval: bool = False
    eval_duration: Duration = field(default_factory=lambda: Duration.epochs(1))
    """Upper bound on each evaluator's pass (steps / tokens / one epoch of its data)."""
    log_interval: int = 5

    def post_attach(self) -> None:
        if not hasattr(self.trainer.train_module, "eval_batch"):
            raise OLMoConfigurationError(f"'{type(self).__name__}' needs a train module with 'eval_batch'")

    def pre_train(self) -> None:
        if self.eval_on_startup:
            self.perform_eval()

    def post_train(self) -> None:
        if self.eval_on_finish:
            self.perform_eval()

    def post_step(self) -> None:
        if self.step <= 1:
            return
        if (self.eval_interval is not None and self.step % self.eval_interval == 0) or (
            self.fixed_steps is not None and self.step in self.fixed_steps
        ):
            self.perform_eval()

    def _progress(self, evaluator: Evaluator, n: int) -> None:
        total = evaluator.total_batches
        log.info(f"[eval={evaluator.name},step={n}" + (f"/{total}]" if total is not None else "]"))

    def perform_eval(self, prefix: str = "eval") -> None:
        """Run every evaluator and record ``{prefix}/{evaluator.name}/{metric}``."""
        if self.trainer.no_evals:
            return
        dp_ws = get_world_size(self.trainer.dp_process_group)
        device = get_default_device()
        timings = []
        for evaluator in self.evaluators:
            log.info(f"Running {evaluator.display_name} evals...")
            start = time.monotonic()
            evaluator.reset_metrics()
            n_batches = n_tokens = 0
            for batch in evaluator:
                n_batches += 1
                n_tokens += batch["input_ids"].numel() * dp_ws
                batch = move_to_device(batch, device)
                with torch.no_grad():
                    out = self.trainer.train_module.eval_batch(batch, labels=get_labels(batch))
                    logits, ce_loss = out.logits, out.ce_loss
                    with cuda_sync_debug_mode(0):
                        evaluator.update_metrics(batch, ce_loss, logits)
                done = self.eval_duration.due(step=n_batches, tokens=n_tokens, epoch=1)
                if done or n_batches % self.log_interval == 0 or n_batches == evaluator.total_batches:
                    self._progress(evaluator, n_batches)
                if done:
                    break
            lines, first = [], None
            with cuda_sync_debug_mode(0):  # one synchronisation per evaluator
                for name, value in evaluator.compute_metrics().items():
                    first = first or name
                    lines.append(f"    {name}={format_float(value.item())}")
                    self.trainer.record_metric(f"{prefix}/{evaluator.name}/{name}", value)
            took = time.monotonic() - start
            timings.append((first or evaluator.name, n_batches, took))
            gc_cuda()
            log.info(f"Finished {evaluator.display_name} evals in {took:.1f} seconds. Metrics:\n" + "\n".join(lines))
        total_t, total_b = sum(t for _, _, t in timings), sum(b for _, b, _ in timings)
        speed = [f"    {name} (+variants): {t:.1f} sec ({b} batches)" for name, b, t in sorted(timings, key=lambda x: x[2])]
        speed.append(f"    Total evaluation time: {total_t:.1f} seconds ({total_b} batches)")
        log.info("Evaluation speed:\n" + "\n".join(speed))
        self.trainer.record_metric("throughput/in-loop eval time (s)", total_t, merge_strategy=MetricMergeStrategy.sum)
        self.trainer.record_metric("throughput/in-loop eval batches", total_b, merge_strategy=MetricMergeStrategy.sum)
        if self.cancel_after_first_eval:
            # every rank gets here at the same time, so no agreement round is needed
            self.trainer.cancel_run("canceled from evaluator callback since 'cancel_after_first_eval' is set", no_sync=True)


def _global_eval_batch_size(spec: EvalBatchSpec, seq_len: int, dp_ws: int) -> int:
    if spec.batch_size_unit == EvalBatchSizeUnit.tokens:
        return spec.rank_batch_size * dp_ws
    if spec.batch_size_unit == EvalBatchSizeUnit.instances:
        return spec.rank_batch_size * seq_len * dp_ws
    raise NotImplementedError(spec.batch_size_unit)


@dataclass
class LMEvaluatorCallbackConfig(CallbackConfig):
    eval_dataset: Any = None
    """A :class:`~olmo_core_b200.data.NumpyDatasetConfig` of a padded fixed-sequence-length dataset with labels."""
    eval_interval: Optional[int] = 1000
    fixed_steps: Optional[List[int]] = None
    eval_on_startup: bool = False
    eval_on_finish: bool = False
    cancel_after_first_eval: bool = False
    eval_duration: Duration = field(default_factory=lambda: Duration.epochs(1))
    log_interval: int = 5
    deterministic: bool = True
    enabled: bool = True

    def build(self, trainer: "Trainer") -> Optional[Callback]:
        if not self.enabled:
            return None
        from ...data import NumpyPaddedFSLDataset

        seq_len = getattr(self.eval_dataset, "max_sequence_length", None) or self.eval_dataset.sequence_length
        spec = trainer.train_module.eval_batch_spec
        if spec.max_sequence_length is not None and seq_len > spec.max_sequence_length:
            raise OLMoConfigurationError(
                f"The maximum sequence length for the LM eval dataset ({seq_len:,d} tokens) is too long for the train "
                f"module's maximum eval sequence length ({spec.max_sequence_length:,d} tokens)"
            )
        dataset = self.eval_dataset.build()
        if not isinstance(dataset, NumpyPaddedFSLDataset):
            raise OLMoConfigurationError(f"Expected a padded FSL dataset, got '{type(dataset).__name__}' instead")
        collator = getattr(trainer.data_loader, "collator", None)
        if collator is None:
            raise OLMoConfigurationError(f"Expected a text data loader with a collator, got '{type(trainer.data_loader).__name__}'")
        evaluator = LMEvaluator.from_numpy_dataset(
            dataset, name="lm", collator=collator, device=trainer.device, dp_process_group=trainer.dp_process_group,
            global_batch_size=_global_eval_batch_size(spec, seq_len, get_world_size(trainer.dp_process_group)),
            deterministic=self.deterministic,
        )
        return EvaluatorCallback(
            evaluators=[evaluator], eval_interval=self.eval_interval, fixed_steps=self.fixed_steps,
            log_interval=self.log_interval, eval_on_startup=self.eval_on_startup, eval_on_finish=self.eval_on_finish,
            cancel_after_first_eval=self.cancel_after_first_eval, eval_duration=self.eval_duration,
        )


@lru_cache(maxsize=1)
def _all_tasks() -> Set[str]:
    from olmo_eval import list_tasks  # optional dependency

    return set(list_tasks())


_METRIC_LABELS = {"f1": "F1 score", "acc": "accuracy", "len_norm": "length-normalized accuracy", "pmi_dc": "PMI-DC accuracy",
                  "ce_loss": "CE loss", "bpb": "BPB", "soft": "soft loss", "soft_log": "log soft loss"}


class DownstreamEvaluator(Evaluator):
    """One in-context-learning task of the ``olmo_eval`` suite; metrics are named ``<task> (<metric label>)``."""

    metric_type_to_label = {f"{k}_v{v}": (label if v == 1 else f"{label} v{v}")
                            for k, label in _METRIC_LABELS.items() for v in (1, 2)}

    def __init__(self, *, name: str, task: str, batch_spec: EvalBatchSpec, tokenizer, device: Optional[torch.device] = None,
                 dp_process_group: Optional[dist.ProcessGroup] = None, lazy: bool = False):
        if task not in _all_tasks():
            raise OLMoConfigurationError(f"Unknown downstream eval task: '{task}'")
        self.label = task
        self.batch_spec = batch_spec
        self.tokenizer = tokenizer
        self.device = device
        self.dp_process_group = dp_process_group
        self.metric = None
        super().__init__(name=name, batches=None if lazy else self._build_data_loader(),
                         batches_factory=self._build_data_loader if lazy else None, device=device)

    @property
    def display_name(self) -> str:
        return f"{self.name} '{self.label}'"

    def _build_data_loader(self):
        from olmo_eval import ICLMetric, build_task
        from torch.utils.data import DataLoader, DistributedSampler

        spec = self.batch_spec
        kwargs: Dict[str, Any] = {}
        if spec.max_sequence_length is not None:
            kwargs["model_ctx_len"] = spec.max_sequence_length
            if spec.fixed_sequence_length:
                kwargs["fixed_ctx_len"] = True
        log.info(f"Building downstream eval task dataset for '{self.label}'...")
        task = build_task(self.label, self.tokenizer, **kwargs)
        self.metric = ICLMetric(metric_type=task.metric_type).to(self.device or get_default_device())
        if spec.max_sequence_length is not None and task.max_sequence_length > spec.max_sequence_length:
            raise OLMoConfigurationError(
                f"The maximum sequence length for downstream eval task '{self.label}' ({task.max_sequence_length:,d} tokens) "
                f"is too long for the train module's maximum eval sequence length ({spec.max_sequence_length:,d} tokens)"
            )
        if spec.batch_size_unit == EvalBatchSizeUnit.instances:
            per_rank = spec.rank_batch_size
        elif spec.batch_size_unit == EvalBatchSizeUnit.tokens:
            per_seq = spec.max_sequence_length if spec.fixed_sequence_length else task.max_sequence_length
            if spec.fixed_sequence_length and spec.rank_batch_size % per_seq != 0:
                raise OLMoConfigurationError(
                    f"The eval batch size ({spec.rank_batch_size} tokens) must be divisible by the maximum eval "
                    f"sequence length ({per_seq:,d} tokens)"
                )
            per_rank = max(spec.rank_batch_size // per_seq, 1)
        else:
            raise NotImplementedError(spec.batch_size_unit)
        sampler = None
        if is_distributed():
            sampler = DistributedSampler(task, drop_last=False, shuffle=False,
                                         num_replicas=get_world_size(self.dp_process_group),
                                         rank=get_rank(self.dp_process_group))
        return DataLoader(task, batch_size=per_rank, collate_fn=task.collate_fn, drop_last=False, shuffle=False,
                          num_workers=0, sampler=sampler)

    def update_metrics(self, batch: Dict[str, Any], ce_loss: Optional[torch.Tensor], logits: Optional[torch.Tensor]) -> None:
        del ce_loss
        if logits is None:
            raise RuntimeError("Downstream evaluators need full logits, which are not gathered under context or tensor "
                               "parallelism; disable downstream evals for such runs.")
        assert self.metric is not None
        self.metric.update(batch, logits)

    def compute_metrics(self) -> Dict[str, torch.Tensor]:
        assert self.metric is not None
        return {f"{self.label} ({self.metric_type_to_label[kind]})": value for kind, value in self.metric.compute().items()}

    def reset_metrics(self) -> None:
        if self.metric is not None:
            self.metric.reset()


@dataclass
class DownstreamEvaluatorCallbackConfig(CallbackConfig):
    tasks: List[str] = field(default_factory=list)
    tokenizer: Any = None
    """A :class:`~olmo_core_b200.data.TokenizerConfig` with an ``identifier``."""
    eval_interval: Optional[int] = 1000
    fixed_steps: Optional[List[int]] = None
    eval_duration: Duration = field(default_factory=lambda: Duration.epochs(1))
    eval_on_startup: bool = False
    eval_on_finish: bool = False
    cancel_after_first_eval: bool = False
    log_interval: int = 5
    lazy: bool = False
    enabled: bool = True

    def build(self, trainer: "Trainer") -> Optional[Callback]:
        if not self.enabled:
            return None
        from olmo_eval import HFTokenizer

        if self.tokenizer is None or self.tokenizer.identifier is None:
            raise OLMoConfigurationError("Tokenizer 'identifier' required to build a concrete tokenizer")
        tok = HFTokenizer(self.tokenizer.identifier, pad_token_id=self.tokenizer.pad_token_id,
                          eos_token_id=self.tokenizer.eos_token_id, bos_token_id=self.tokenizer.bos_token_id)
        evaluators: List[Evaluator] = [
            DownstreamEvaluator(name="downstream", task=task, batch_spec=trainer.train_module.eval_batch_spec, tokenizer=tok,
                                device=trainer.device, dp_process_group=trainer.dp_process_group, lazy=self.lazy)
            for task in sorted(self.tasks)
        ]
        return EvaluatorCallback(
            evaluators=evaluators, eval_interval=self.eval_interval, fixed_steps=self.fixed_steps,
            eval_on_startup=self.eval_on_startup, eval_on_finish=self.eval_on_finish, log_interval=self.log_interval,
            cancel_after_first_eval=self.cancel_after_first_eval, eval_duration=self.eval_duration,
        )
