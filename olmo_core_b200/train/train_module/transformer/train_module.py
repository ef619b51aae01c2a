"""
Train module for transformer language models
(API of src/olmo_core/train/train_module/transformer/train_module.py:65-657).

One training step = micro-batches of ``rank_microbatch_size`` tokens, each a forward + backward whose weight
gradients accumulate into the sharded-parameter runtime's fp32 ``main_grad`` buffer from the wgrad GEMM
epilogues; then ``optim_step``: one gradient reduce-scatter, global grad-norm (device scalar), clipping
coefficient and skip-step factor folded into the fused AdamW kernel, one bf16 all-gather.

Loss normalisation follows the reference: the CE of every micro-batch is *summed* and divided by the number
of target tokens in the rank's whole batch; gradients are then averaged over data-parallel ranks.
"""

from __future__ import annotations

import contextlib
import logging
from functools import lru_cache
from typing import Any, Dict, Generator, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ....data.utils import get_labels, split_batch
from ....distributed.parallel import build_world_mesh, get_dp_process_group, get_world_mesh
from ....distributed.utils import get_reduce_divide_factor, get_world_size, is_distributed
from ....exceptions import OLMoConfigurationError
from ....float8 import Float8Config
from ....nn.lm_head import LMOutputWithLoss
from ....nn.transformer import MoETransformer, NormalizedTransformer, Transformer
from ....optim import OptimConfig, SkipStepOptimizer
from ....optim.scheduler import Scheduler
from ....utils import gc_cuda, get_default_device, move_to_device
from ...common import MetricMergeStrategy, ReduceType
from ..train_module import EvalBatchSpec, TrainModule
from .common import parallelize_model
from .config import (
    TransformerActivationCheckpointingConfig,
    TransformerContextParallelConfig,
    TransformerDataParallelConfig,
    TransformerExpertParallelConfig,
    TransformerTensorParallelConfig,
)

log = logging.getLogger(__name__)

__all__ = ["TransformerTrainModule"]


class TransformerTrainModule(TrainModule):
    def __init__(
        self,
        model: Transformer,
        optim: OptimConfig,
        rank_microbatch_size: int,
        max_sequence_length: int,
        compile_model: bool = False,
        float8_config: Optional[Float8Config] = None,
        dp_config: Optional[TransformerDataParallelConfig] = None,
        tp_config: Optional[TransformerTensorParallelConfig] = None,
        cp_config: Optional[TransformerContextParallelConfig] = None,
        ep_config: Optional[TransformerExpertParallelConfig] = None,
        ac_config: Optional[TransformerActivationCheckpointingConfig] = None,
        z_loss_multiplier: Optional[float] = None,
        autocast_precision: Optional[torch.dtype] = None,
        max_grad_norm: Optional[float] = None,
        scheduler: Optional[Scheduler] = None,
        device: Optional[torch.device] = None,
        state_dict_save_opts: Optional[Dict[str, Any]] = None,
        state_dict_load_opts: Optional[Dict[str, Any]] = None,
        load_key_mapping: Optional[Dict[str, str]] = None,
        label_ignore_index: int = -100,
    ):
        super().__init__()
        if rank_microbatch_size % max_sequence_length != 0:
            raise OLMoConfigurationError(
                f"'rank_microbatch_size' ({rank_microbatch_size:,d} tokens) must be divisible by "
                f"'max_sequence_length' ({max_sequence_length:,d} tokens)"
            )
        self.device = device or get_default_device()
        self.world_mesh = None
        if is_distributed():
            self.world_mesh = get_world_mesh()
            if self.world_mesh is None:
                self.world_mesh = build_world_mesh(dp=dp_config, tp=tp_config, cp=cp_config, ep=ep_config,
                                                   device_type=self.device.type)
        elif any(c is not None for c in (dp_config, tp_config, cp_config, ep_config)) and False:
            raise OLMoConfigurationError("Training parallelism configs are only valid for distributed training")

        self.model = parallelize_model(
            model,
            world_mesh=self.world_mesh,
            device=self.device,
            max_sequence_length=max_sequence_length,
            rank_microbatch_size=rank_microbatch_size,
            compile_model=compile_model,
            float8_config=float8_config,
            dp_config=dp_config,
            tp_config=tp_config,
            cp_config=cp_config,
            ep_config=ep_config,
            ac_config=ac_config,
        )
        self._dp_config = dp_config
        self._cp_config = cp_config
        self._tp_config = tp_config
        self._ep_config = ep_config
        self.label_ignore_index = label_ignore_index
        self.z_loss_multiplier = z_loss_multiplier
        self.rank_microbatch_size = rank_microbatch_size
        self.max_sequence_length = max_sequence_length
        self.autocast_precision = autocast_precision
        self.max_grad_norm = max_grad_norm
        self.scheduler = scheduler
        self.state_dict_save_opts = state_dict_save_opts or {}
        self.state_dict_load_opts = state_dict_load_opts or {}
        self.load_key_mapping = load_key_mapping
        self.runtime = getattr(self.model, "_sharding_runtime", None)

        log.info("Building optimizer...")
        self.optim = optim.build(self.model, strict=True)
        self._grad_scale = torch.ones((), dtype=torch.float32, device=self.device)

    # -- properties ------------------------------------------------------------------------------------------
    @property
    def dp_process_group(self) -> Optional[dist.ProcessGroup]:
        return None if self.world_mesh is None else get_dp_process_group(self.world_mesh)

    @property
    def eval_batch_spec(self) -> EvalBatchSpec:
        return EvalBatchSpec(self.rank_microbatch_size, max_sequence_length=self.max_sequence_length)

    @property
    def dp_config(self) -> Optional[TransformerDataParallelConfig]:
        return self._dp_config

    @property
    def tp_enabled(self) -> bool:
        return self._tp_config is not None

    @property
    def cp_enabled(self) -> bool:
        return self._cp_config is not None

    @property
    def ep_enabled(self) -> bool:
        return self._ep_config is not None

    def pre_train(self) -> None:
        dp_ws = get_world_size(self.trainer.dp_process_group)
        if self.trainer.global_batch_size % (self.rank_microbatch_size * dp_ws) != 0:
            raise OLMoConfigurationError(
                f"global batch size ({self.trainer.global_batch_size:,d}) must be divisible by "
                f"micro-batch size ({self.rank_microbatch_size:,d}) x DP world size ({dp_ws})"
            )

    # -- state dicts -------------------------------------------------------------------------------------------
    def _named_params(self) -> Dict[str, nn.Parameter]:
        return dict(self.model.named_parameters())

    def _present(self, name: str, p: torch.Tensor, local: torch.Tensor) -> torch.Tensor:
        if self.runtime is not None:
            slot = self.runtime.slot_for(p)
            if slot is not None:
                return self.runtime.sharded_tensor(slot, local)
        return local

    def state_dict(self, *, optim: Optional[bool] = None, flatten_optimizer_state: bool = True) -> Dict[str, Any]:
        """
        ``{"model": {fqn: tensor}, "optim": {"state.<fqn>.<field>": tensor, "param_groups.<fqn>.<field>": value}}``.
        Sharded tensors are presented as dim-0 ``DTensor`` shards so that the checkpoint layer writes the same
        per-parameter shards, under the same keys, as the reference's flattened optimizer state dicts. With
        ``flatten_optimizer_state=False`` the param groups are one list of dicts instead (the layout the reference
        writes when flattening is off; on disk ``optim.param_groups.<i>.<field>``).
        """
        optim = True if optim is None else optim
        if optim and not flatten_optimizer_state:
            from ....distributed.checkpoint import optim_state

            sd = self.state_dict(optim=False)
            sd["optim"] = optim_state(self.model, self.optim, flatten=False)
            return sd
        params = self._named_params()
        sd: Dict[str, Any] = {"model": {n: self._present(n, p, p.data) for n, p in params.items()}}
        for n, b in self.model.named_buffers():
            if n.split(".")[-1] not in getattr(self.model, "_non_persistent_buffers_set", set()):
                sd["model"].setdefault(n, b)
        if optim:
            osd: Dict[str, Any] = {}
            name_of = {id(p): n for n, p in params.items()}
            for group in self.optim.param_groups:
                for p in group["params"]:
                    n = name_of.get(id(p))
                    if n is None:
                        continue
                    for field, value in self.optim.state.get(p, {}).items():
                        if torch.is_tensor(value) and value.dim() > 0:
                            value = self._present(n, p, value)
                        osd[f"state.{n}.{field}"] = value
                    for field, value in group.items():
                        if field != "params":
                            osd[f"param_groups.{n}.{field}"] = value
            sd["optim"] = osd
        return sd

    def state_dict_to_save(self, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        return self.state_dict(optim=optim)

    def state_dict_to_load(self, metadata, *, optim: Optional[bool] = None) -> Dict[str, Any]:
        keys = set(getattr(metadata, "state_dict_metadata", {}).keys()) if metadata is not None else set()
        has_optim = any(k.startswith("optim.") for k in keys)
        if optim is None:
            optim = has_optim
        elif optim and not has_optim:
            raise RuntimeError("Checkpoint does not contain optimizer state, but 'optim=True' was requested")
        if optim:
            self._ensure_optim_state()
        # the checkpoint decides the optimizer-state layout (the reference switches the same way:
        # src/olmo_core/train/train_module/transformer/train_module.py:278-293)
        flat = "optim.param_groups.0.params" not in keys
        sd = self.state_dict(optim=optim, flatten_optimizer_state=flat)
        if self.load_key_mapping is not None:
            from ....distributed.checkpoint import swap_param_keys

            swap_param_keys(sd, self.load_key_mapping, metadata=metadata)
        if not self.state_dict_load_opts.get("strict", True) and keys:
            from ....distributed.checkpoint import prune_state_dict

            pruned = prune_state_dict(sd, keys)
            if pruned:
                log.warning(f"Checkpoint is missing the following keys: {pruned}")
        return sd

    def _ensure_optim_state(self) -> None:
        """Materialise optimizer state tensors so that they can be loaded into in place."""
        if hasattr(self.optim, "_init_flat_state") and self.runtime is not None:
            self.optim._init_flat_state()
            return
        for group in self.optim.param_groups:
            for p in group["params"]:
                st = self.optim.state[p]
                if not st and p.requires_grad:
                    st["step"] = torch.zeros((), dtype=torch.float32, device=p.device)
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        from ....distributed.utils import get_local_tensor

        if self.load_key_mapping is not None:
            from ....distributed.checkpoint import swap_param_keys

            swap_param_keys(state_dict, self.load_key_mapping, reverse=True, quiet=True)
        params = self._named_params()
        strict = self.state_dict_load_opts.get("strict", True)
        with torch.no_grad():
            for n, value in state_dict["model"].items():
                target = params.get(n)
                if target is None:
                    bufs = dict(self.model.named_buffers())
                    if n in bufs:
                        bufs[n].copy_(get_local_tensor(value))
                    elif strict:
                        raise KeyError(f"unexpected key '{n}' in model state dict")
                    continue
                src = get_local_tensor(value)
                if src.data_ptr() != target.data.data_ptr():
                    target.data.copy_(src)
            if "optim" in state_dict:
                self._ensure_optim_state()
                name_of = {id(p): n for n, p in params.items()}
                osd = state_dict["optim"]
                if isinstance(osd.get("param_groups"), list):  # unflattened layout
                    for group, saved in zip(self.optim.param_groups, osd["param_groups"]):
                        for field, value in saved.items():
                            if field not in ("params", "initial_lr") and field in group:
                                group[field] = value
                for group in self.optim.param_groups:
                    for p in group["params"]:
                        n = name_of.get(id(p))
                        if n is None:
                            continue
                        for field, cur in self.optim.state.get(p, {}).items():
                            key = f"state.{n}.{field}"
                            if key in osd and torch.is_tensor(cur):
                                src = get_local_tensor(osd[key]) if torch.is_tensor(osd[key]) else torch.tensor(osd[key])
                                if src.data_ptr() != cur.data_ptr():
                                    cur.copy_(src.to(cur.device))
                        for field in list(group.keys()):
                            key = f"param_groups.{n}.{field}"
                            if field != "params" and key in osd and field not in ("initial_lr",):
                                group[field] = osd[key]
        if self.runtime is not None:
            self.runtime.sync_lowp()
        gc_cuda()

    # -- training ------------------------------------------------------------------------------------------------
    def zero_grads(self) -> None:
        if self.runtime is not None:
            self.runtime.zero_grad()
        self.optim.zero_grad(set_to_none=True)

    def model_forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None, **kwargs):
        with self._model_forward_context():
            return self.model(input_ids=input_ids, labels=labels, **kwargs)

    def train_batch(self, batch: Dict[str, Any], dry_run: bool = False) -> None:
        self.model.train()
        if "labels" not in batch:
            batch["labels"] = get_labels(batch, label_ignore_index=self.label_ignore_index)
        # total target tokens of this rank's batch; the loss of every micro-batch is divided by it
        batch_num_tokens_for_loss = move_to_device((batch["labels"] != self.label_ignore_index).sum(), self.device)
        total_tokens = batch["labels"].numel()
        if not dry_run and total_tokens > 0:
            # both metrics are proportions in [0, 1]; the names are the ones dashboards built on the reference expect
            self.record_metric("train/masked labels (%)", 1.0 - batch_num_tokens_for_loss / total_tokens, ReduceType.mean)
        instance_mask = batch.get("instance_mask")
        if instance_mask is not None:
            dropped = move_to_device((~instance_mask).sum(), self.device)
            if not dry_run:
                self.record_metric("train/masked instances (%)", dropped / max(instance_mask.numel(), 1), ReduceType.mean)
            # Instances removed by the instance filter still count, with zero loss, towards the divisor: every rank then
            # divides by the token count of a full batch whatever the filter dropped locally, which keeps the ranks'
            # contributions comparable without a collective (same convention as the reference:
            # src/olmo_core/train/train_module/transformer/train_module.py:368-380).
            batch_num_tokens_for_loss = batch_num_tokens_for_loss + dropped * batch["labels"].shape[1]
        ce_batch_loss = torch.zeros((), dtype=torch.float32, device=self.device)
        z_batch_loss = torch.zeros((), dtype=torch.float32, device=self.device) if self.z_loss_multiplier is not None else None

        seq_len = batch["input_ids"].shape[1]
        micro_batches = split_batch(batch, max(1, self.rank_microbatch_size // seq_len))
        for idx, mb in enumerate(micro_batches):
            with self._train_microbatch_context(idx, len(micro_batches)):
                input_ids, labels, model_kwargs = self._prepare_batch(mb)
                out = self.model_forward(
                    input_ids, labels=labels, ignore_index=self.label_ignore_index, loss_reduction="sum",
                    z_loss_multiplier=self.z_loss_multiplier, loss_div_factor=batch_num_tokens_for_loss,
                    return_logits=False, **model_kwargs,
                )
                assert isinstance(out, LMOutputWithLoss)
                ce_batch_loss += out.ce_loss.detach().float()
                if z_batch_loss is not None and out.z_loss is not None:
                    z_batch_loss += out.z_loss.detach().float()
                out.loss.backward()
        del batch

        self.model.post_batch(dry_run=dry_run)
        if dry_run:
            if isinstance(self.model, MoETransformer):
                self.model.reset_auxiliary_metrics()
            return

        if isinstance(self.optim, SkipStepOptimizer):
            # the skip decision needs the global loss: mean over all ranks, pre-divided for fp safety
            loss_for_skip = ce_batch_loss.clone()
            if is_distributed():
                f = get_reduce_divide_factor(get_world_size())
                loss_for_skip.div_(f)
                dist.all_reduce(loss_for_skip)
                loss_for_skip.div_(get_world_size()).mul_(f)
            self.optim.latest_loss = loss_for_skip

        self.latest_ce_loss = ce_batch_loss
        self.record_ce_loss(ce_batch_loss, ReduceType.mean)
        if z_batch_loss is not None:
            self.record_metric("Z loss", z_batch_loss, ReduceType.mean, namespace="train")
            self.record_metric("Z loss unscaled", z_batch_loss / self.z_loss_multiplier, ReduceType.mean, namespace="train")
        if isinstance(self.model, MoETransformer):
            for name, (value, reduce_type) in self.model.compute_auxiliary_metrics(reset=True).items():
                self.record_metric(name, value, reduce_type, namespace="train", merge_strategy=MetricMergeStrategy.sum)

    def eval_batch(self, batch: Dict[str, Any], labels: Optional[torch.Tensor] = None):
        self.model.eval()
        input_ids, labels_, kwargs = self._prepare_batch(batch, labels)
        with torch.no_grad(), self._model_forward_context():
            return self.model(input_ids=input_ids, labels=labels_, ignore_index=self.label_ignore_index,
                              loss_reduction="none", return_logits=True, **kwargs)

    def optim_step(self) -> None:
        rt = self.runtime
        if rt is not None:
            rt.reduce_gradients()
        if self.max_grad_norm is not None or isinstance(self.optim, SkipStepOptimizer):
            grad_norm = self._grad_norm()
            self.record_metric("total grad norm", grad_norm, reduce_type=None, namespace="optim")
            if isinstance(self.optim, SkipStepOptimizer):
                self.optim.latest_grad_norm = grad_norm
            if self.max_grad_norm is not None:
                self._apply_clip(grad_norm)
        if self.scheduler is not None:
            for i, group in enumerate(self.optim.param_groups):
                new_lr = self.scheduler.set_lr(group, self.trainer)
                self.record_metric(f"LR (group {i})", new_lr, namespace="optim")
        self.optim.step()
        if isinstance(self.optim, SkipStepOptimizer):
            self.record_metric("step skipped", self.optim.step_skipped, namespace="optim")
        self.model.post_optim_step()

    def _grad_norm(self) -> torch.Tensor:
        if self.runtime is not None:
            return self.runtime.grad_norm_sq().sqrt()
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        if not grads:
            return torch.zeros((), device=self.device)
        return torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float()) for g in grads]))

    def _apply_clip(self, grad_norm: torch.Tensor) -> None:
        """``min(1, max_norm / (norm + 1e-6))``, folded into the optimizer kernel when it accepts a grad scale."""
        coef = torch.clamp(self.max_grad_norm / (grad_norm + 1e-6), max=1.0)
        if hasattr(self.optim, "grad_scale"):
            self._grad_scale.copy_(coef)
            self.optim.grad_scale = self._grad_scale
            return
        if self.runtime is not None and self.runtime.grad_shard is not None:
            self.runtime.grad_shard.mul_(coef)
        elif self.runtime is not None and self.runtime.main_grad is not None:
            self.runtime.main_grad.mul_(coef)
        for p in self.model.parameters():
            if p.grad is not None:
                p.grad.mul_(coef.to(p.grad.dtype))

    # -- helpers -----------------------------------------------------------------------------------------------------
    def _prepare_batch(self, batch: Dict[str, Any], labels: Optional[torch.Tensor] = None
                       ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Dict[str, Any]]:
        input_ids = batch["input_ids"]
        labels = labels if labels is not None else batch.get("labels")
        kwargs = {k: v for k, v in batch.items() if k in ("doc_lens", "max_doc_lens")}
        if not self.cp_enabled:
            input_ids = move_to_device(input_ids, self.device)
            labels = move_to_device(labels, self.device) if labels is not None else None
        return input_ids, labels, kwargs

    @contextlib.contextmanager
    def _train_microbatch_context(self, micro_batch_idx: int, num_micro_batches: int) -> Generator[None, None, None]:
        # Gradients accumulate locally in main_grad across micro-batches; the cross-rank reduction belongs to the last
        # one: the runtime starts it block by block behind that micro-batch's backward and finishes it in optim_step().
        begin = getattr(self.runtime, "begin_microbatch", None)
        if begin is not None:
            begin(micro_batch_idx, num_micro_batches)
        yield

    @contextlib.contextmanager
    def _model_forward_context(self) -> Generator[None, None, None]:
        if self.autocast_precision is not None:
            with torch.autocast(self.device.type, dtype=self.autocast_precision):
                yield
        else:
            yield

    @lru_cache
    def num_flops_per_token(self, seq_len: int) -> Optional[int]:
        return self.model.num_flops_per_token(seq_len)

    def global_num_flops_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        seq_len = batch["input_ids"].shape[1]
        per_tok = self.num_flops_per_token(seq_len)
        if per_tok is None:
            return None
        return per_tok * self.trainer.data_loader.global_num_tokens_in_batch(batch)
