"""
Train module for pipeline-parallel transformers
(role of src/olmo_core/train/train_module/transformer/pipeline_train_module.py:68-701): the model is cut into
stages, each rank owns one or more stages with their own optimizer, micro-batches flow through a
``torch.distributed.pipelining`` schedule whose stage-to-stage transfers are NCCL point-to-point.
"""

from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ....data.utils import get_labels
from ....distributed.parallel import PipelineSchedule, build_world_mesh, get_dp_process_group, get_pp_mesh, get_world_mesh
from ....distributed.utils import get_world_size
from ....exceptions import OLMoConfigurationError
from ....nn.functional import cross_entropy_loss
from ....optim import OptimConfig, SkipStepOptimizer
from ....utils import get_default_device, move_to_device
from ...common import ReduceType
from ..train_module import EvalBatchSpec, TrainModule
from .common import parallelize_model

log = logging.getLogger(__name__)

__all__ = ["TransformerPipelineTrainModule"]


class TransformerPipelineTrainModule(TrainModule):
    def __init__(self, model, optim: OptimConfig, rank_microbatch_size: int, max_sequence_length: int, pp_config,
                 compile_model: bool = False, float8_config=None, dp_config=None, tp_config=None, cp_config=None,
                 ep_config=None, ac_config=None, z_loss_multiplier: Optional[float] = None,
                 autocast_precision: Optional[torch.dtype] = None, max_grad_norm: Optional[float] = None,
                 scheduler=None, device: Optional[torch.device] = None, state_dict_save_opts=None,
                 state_dict_load_opts=None, load_key_mapping=None, label_ignore_index: int = -100):
        super().__init__()
        if cp_config is not None or ep_config is not None:
            raise OLMoConfigurationError("context / expert parallelism are not supported together with pipeline parallelism")
        self.device = device or get_default_device()
        self.world_mesh = get_world_mesh() or build_world_mesh(dp=dp_config, tp=tp_config, pp=pp_config,
                                                               device_type=self.device.type)
        self.pp_config = pp_config
        self._tp_config, self._cp_config = tp_config, cp_config
        self.pp_mesh = get_pp_mesh(self.world_mesh)
        self.rank_microbatch_size = rank_microbatch_size
        self.max_sequence_length = max_sequence_length
        self.z_loss_multiplier = z_loss_multiplier
        self.max_grad_norm = max_grad_norm
        self.scheduler = scheduler
        self.label_ignore_index = label_ignore_index
        stages, parts = pp_config.split_model(model, pp_mesh=self.pp_mesh, device=self.device)
        self.model_parts: List[Any] = []
        for i, part in enumerate(parts):
            self.model_parts.append(parallelize_model(
                part, world_mesh=self.world_mesh, device=self.device, max_sequence_length=max_sequence_length,
                rank_microbatch_size=rank_microbatch_size, compile_model=compile_model, float8_config=float8_config,
                dp_config=dp_config, tp_config=tp_config, ac_config=ac_config, pp_enabled=True))
        self._stages = stages
        self.optimizers = [optim.build(p, strict=False) for p in self.model_parts]
        self._schedule: Optional[PipelineSchedule] = None
        self._batch_tokens_for_loss: Optional[torch.Tensor] = None

    @property
    def dp_process_group(self):
        return get_dp_process_group(self.world_mesh)

    @property
    def eval_batch_spec(self) -> EvalBatchSpec:
        return EvalBatchSpec(self.rank_microbatch_size, max_sequence_length=self.max_sequence_length)

    @property
    def tp_enabled(self) -> bool:
        return self._tp_config is not None

    @property
    def cp_enabled(self) -> bool:
        return self._cp_config is not None

    @property
    def train_pp_schedule(self) -> PipelineSchedule:
        """The schedule of the current batch shape; it exists once a batch has been seen."""
        if self._schedule is None:
            raise RuntimeError("the pipeline schedule is built by the first training batch")
        return self._schedule

    def loss_fn(self, output: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """Loss of the last stage's output for one micro-batch, already divided by the batch's target count."""
        return self._loss_fn(output, labels)

    def run_pipeline(self, input_ids: torch.Tensor, labels: torch.Tensor, batch_num_tokens_for_loss, **kwargs):
        """
        One pass of the schedule over the batch (forward and backward of every micro-batch). Returns the summed loss
        on ranks that hold the last stage, ``None`` elsewhere
        (reference: src/olmo_core/train/train_module/transformer/pipeline_train_module.py:552-609).
        """
        if not torch.is_tensor(batch_num_tokens_for_loss):
            batch_num_tokens_for_loss = torch.tensor(float(batch_num_tokens_for_loss))
        self._batch_tokens_for_loss = move_to_device(batch_num_tokens_for_loss, self.device)
        seq_len = input_ids.shape[1]
        n_mb = max(1, input_ids.shape[0] // max(1, self.rank_microbatch_size // seq_len))
        _, loss = self._get_schedule(n_mb).step(input_ids, target=labels, **kwargs)
        return loss

    def reduce_send_recv(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """
        Make a scalar that only the last stage's ranks hold known to every rank: those ranks pass it in and it is
        averaged over their data-parallel group; the others pass ``None``. One sum over the pipeline group then
        delivers it (reference: pipeline_train_module.py:465-504, which relays it stage by stage instead).
        """
        if x is None:
            x = torch.zeros((), device=self.device)
        else:
            x = x.detach().clone().to(self.device)
            group = self.dp_process_group
            if group is not None and dist.get_world_size(group) > 1:
                dist.all_reduce(x, group=group)
                x.div_(dist.get_world_size(group))
        dist.all_reduce(x, group=self.pp_mesh.get_group())
        return x

    def _loss_fn(self, logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        ce, z = cross_entropy_loss(logits.view(-1, logits.size(-1)), labels.view(-1), ignore_index=self.label_ignore_index,
                                   reduction="sum", compute_z_loss=self.z_loss_multiplier is not None,
                                   z_loss_multiplier=self.z_loss_multiplier or 1e-4)
        loss = ce if z is None else ce + z
        return loss / self._batch_tokens_for_loss

    def _get_schedule(self, num_microbatches: int) -> PipelineSchedule:
        if self._schedule is None or self._schedule.num_microbatches != num_microbatches:
            self._schedule = PipelineSchedule(model_parts=self.model_parts, stages=self._stages, pp_mesh=self.pp_mesh,
                                              schedule_name=self.pp_config.schedule, loss_fn=self._loss_fn,
                                              num_microbatches=num_microbatches)
        return self._schedule

    def state_dict(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        """
        The same layout as the non-pipelined train module writes: ``model.<fqn>`` and, flattened,
        ``optim.state.<fqn>.<field>`` / ``optim.param_groups.<fqn>.<field>``, with sharded tensors presented as dim-0
        ``DTensor`` shards. Every rank contributes the parameters of its own stages; block names keep their global
        index, so a checkpoint written with one pipeline layout loads with another, or without pipelining
        (reference: src/olmo_core/train/train_module/transformer/pipeline_train_module.py:343).
        """
        from ....distributed.checkpoint import model_state, optim_state

        sd: Dict[str, Any] = {"model": {}}
        if optim is not False:
            sd["optim"] = {}
        for part, opt in zip(self.model_parts, self.optimizers):
            sd["model"].update(model_state(part))
            if optim is not False:
                sd["optim"].update(optim_state(part, opt, flatten=True))
        return sd

    def state_dict_to_save(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        return self.state_dict(optim=optim)

    def state_dict_to_load(self, metadata, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        from ....distributed.checkpoint import _ensure_optim_state

        keys = set(getattr(metadata, "state_dict_metadata", {}).keys()) if metadata is not None else set()
        has_optim = any(k.startswith("optim.") for k in keys)
        if optim is None:
            optim = has_optim
        elif optim and not has_optim:
            raise RuntimeError("Checkpoint does not contain optimizer state, but 'optim=True' was requested")
        if optim:
            for part, opt in zip(self.model_parts, self.optimizers):
                _ensure_optim_state(part, opt)
        return self.state_dict(optim=optim)

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        from ....distributed.checkpoint import load_model_state, load_optim_state

        for part, opt in zip(self.model_parts, self.optimizers):
            names = {n for n, _ in part.named_parameters()} | {n for n, _ in part.named_buffers()}
            load_model_state(part, {k: v for k, v in state_dict["model"].items() if k in names}, strict=False)
            if "optim" in state_dict:
                load_optim_state(part, opt, state_dict["optim"])

    def train_batch(self, batch: Dict[str, Any], dry_run: bool = False) -> None:
        for p in self.model_parts:
            p.train()
        if "labels" not in batch:
            batch["labels"] = get_labels(batch, self.label_ignore_index)
        input_ids = move_to_device(batch["input_ids"], self.device)
        labels = move_to_device(batch["labels"], self.device)
        loss = self.run_pipeline(input_ids, labels, (batch["labels"] != self.label_ignore_index).sum())
        if dry_run:
            return
        # The loss lives on the rank with the last stage: average over DP there, then hand it down the pipe.
        value = loss.detach() if loss is not None else torch.zeros((), device=self.device)
        pp_group = self.pp_mesh.get_group()
        dist.all_reduce(value, group=pp_group)  # only the last-stage rank contributes a non-zero value
        self.latest_ce_loss = value
        self.record_ce_loss(value, ReduceType.mean)
        for opt in self.optimizers:
            if isinstance(opt, SkipStepOptimizer):
                opt.latest_loss = value

    def eval_batch(self, batch: Dict[str, Any], labels: Optional[Any] = None) -> Any:
        raise NotImplementedError("evaluation is not supported with pipeline parallelism")

    def optim_step(self) -> None:
        norms_sq = torch.zeros((), device=self.device)
        for part in self.model_parts:
            rt = getattr(part, "_sharding_runtime", None)
            if rt is not None:
                rt.reduce_gradients()
                norms_sq += rt.grad_norm_sq()
            else:
                for p in part.parameters():
                    if p.grad is not None:
                        norms_sq += p.grad.float().pow(2).sum()
        dist.all_reduce(norms_sq, group=self.pp_mesh.get_group())
        grad_norm = norms_sq.sqrt()
        self.record_metric("total grad norm", grad_norm, namespace="optim")
        coef = None
        if self.max_grad_norm is not None:
            coef = torch.clamp(self.max_grad_norm / (grad_norm + 1e-6), max=1.0)
        for opt in self.optimizers:
            if isinstance(opt, SkipStepOptimizer):
                opt.latest_grad_norm = grad_norm
            if coef is not None and hasattr(opt, "grad_scale"):
                opt.grad_scale = coef
            if self.scheduler is not None:
                for group in opt.param_groups:
                    self.scheduler.set_lr(group, self.trainer)
            opt.step()
        for part in self.model_parts:
            part.post_optim_step()

    def zero_grads(self) -> None:
        for part, opt in zip(self.model_parts, self.optimizers):
            rt = getattr(part, "_sharding_runtime", None)
            if rt is not None:
                rt.zero_grad()
            opt.zero_grad(set_to_none=True)

    def num_flops_per_token(self, seq_len: int) -> Optional[int]:
        return sum(p.num_flops_per_token(seq_len) for p in self.model_parts)

    def global_num_flops_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        # every PP rank holds a slice of the model; the per-device share is accounted by the speed monitor
        return self.num_flops_per_token(batch["input_ids"].shape[1]) * self.trainer.data_loader.global_num_tokens_in_batch(batch)
