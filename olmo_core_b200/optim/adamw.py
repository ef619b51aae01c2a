"""
AdamW and SkipStep-AdamW (API of src/olmo_core/optim/adamw.py:12-291).

:class:`SkipStepAdamW` runs the update with the kernel in ``ops/csrc/elementwise.cu`` (one pass over
p, m, v, g; optional bf16 write-back). When the model is managed by the sharded-parameter runtime the
optimizer works directly on the runtime's flat buffers: gradients come from the reduce-scattered fp32 shard,
the clipping coefficient and the skip-step factor are device scalars consumed inside the kernel, and the
kernel writes the updated bf16 rows straight into the resident compute copy that the next all-gather
distributes -- the "cast + scale + partitioned AdamW" tail of the gradient reduce-scatter.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Type, Union

import torch

from ..config import DType
from ..distributed.utils import get_local_tensor
from ..ops.optim import adamw_step_
from .config import OptimConfig
from .skip_step_optimizer import SkipStepOptimizer

__all__ = ["adamw_step", "foreach_adamw_step", "SkipStepAdamW", "AdamWConfig", "SkipStepAdamWConfig"]


def adamw_step(
    p: torch.Tensor,
    grad: torch.Tensor,
    *,
    lr: float,
    betas: Tuple[float, float],
    eps: float,
    weight_decay: float,
    exp_avg: torch.Tensor,
    exp_avg_sq: torch.Tensor,
    step: torch.Tensor,
    step_factor: torch.Tensor,
    step_increment_bugfix: bool = True,
    grad_scale: Optional[torch.Tensor] = None,
    lowp: Optional[torch.Tensor] = None,
) -> None:
    """One SkipStep-AdamW update of a single tensor (decoupled weight decay, bias-corrected moments)."""
    adamw_step_(p, exp_avg, exp_avg_sq, grad, lr=float(lr), betas=betas, eps=eps, weight_decay=weight_decay,
                step=step if step_increment_bugfix else torch.zeros_like(step), step_factor=step_factor,
                grad_scale=grad_scale, lowp=lowp)
    if step_increment_bugfix:
        step.add_(step_factor.to(step.dtype))


def foreach_adamw_step(params: List[torch.Tensor], grads: List[torch.Tensor], exp_avgs: List[torch.Tensor],
                       exp_avg_sqs: List[torch.Tensor], steps: List[torch.Tensor], **kwargs) -> None:
    """Multi-tensor form: on CUDA each tensor is one fused kernel launch."""
    for p, g, m, v, s in zip(params, grads, exp_avgs, exp_avg_sqs, steps):
        adamw_step(p, g, exp_avg=m, exp_avg_sq=v, step=s, **kwargs)


class SkipStepAdamW(SkipStepOptimizer):
    def __init__(
        self,
        params,
        lr: float = 1e-3,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
        rolling_interval_length: int = 128,
        sigma_factor: int = 6,
        dtype: Optional[Union[torch.dtype, DType]] = None,
        foreach: bool = False,
        step_increment_bugfix: bool = True,
    ) -> None:
        assert lr >= 0.0
        assert all(0.0 <= b <= 1.0 for b in betas)
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay),
                         rolling_interval_length=rolling_interval_length, sigma_factor=sigma_factor)
        self.dtype = dtype.as_pt() if isinstance(dtype, DType) else dtype
        self.foreach = foreach
        self.stepfix = step_increment_bugfix
        self._step_skipped: Optional[torch.Tensor] = None
        self._runtime = None
        self._flat_m: Optional[torch.Tensor] = None
        self._flat_v: Optional[torch.Tensor] = None
        self.grad_scale: Optional[torch.Tensor] = None  # clipping coefficient, set by the train module
        self.skip_enabled = True

    # -- flat fast path --------------------------------------------------------------------------------
    def attach_runtime(self, runtime) -> None:
        """Use the sharded-parameter runtime's flat buffers for parameters, gradients and moments."""
        self._runtime = runtime
        if not runtime.materialized:
            return
        self._init_flat_state()

    def _init_flat_state(self) -> None:
        rt = self._runtime
        if self._flat_m is not None or rt is None or rt.master is None:
            return
        self._flat_m = torch.zeros_like(rt.master)
        self._flat_v = torch.zeros_like(rt.master)
        for slot in rt.slots:
            p = slot.param
            if not p.requires_grad:
                continue
            sl = slice(slot.master_offset, slot.master_offset + slot.local_numel)
            self.state[p] = {
                "step": torch.zeros((), dtype=torch.float32, device=rt.master.device),
                "exp_avg": self._flat_m[sl].view(p.shape),
                "exp_avg_sq": self._flat_v[sl].view(p.shape),
            }

    @property
    def step_skipped(self) -> torch.Tensor:
        return self._step_skipped if self._step_skipped is not None else torch.tensor(0.0)

    def _factor(self) -> torch.Tensor:
        if not self.skip_enabled:
            return torch.ones((), dtype=torch.float32, device=self.device)
        return self.get_step_factor()

    @torch.no_grad()
    def step(self, closure=None) -> None:
        if closure is not None:
            with torch.enable_grad():
                closure()
        f = self._factor()
        self._step_skipped = 1 - f
        rt = self._runtime
        if rt is not None and rt.materialized:
            self._init_flat_state()
            self._step_flat(f)
            return
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = torch.zeros((), dtype=torch.float32, device=p.device)
                    state["exp_avg"] = torch.zeros_like(p, dtype=self.dtype)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=self.dtype)
                adamw_step(get_local_tensor(p), get_local_tensor(p.grad), lr=group["lr"], betas=group["betas"],
                           eps=group["eps"], weight_decay=group["weight_decay"],
                           exp_avg=get_local_tensor(state["exp_avg"]), exp_avg_sq=get_local_tensor(state["exp_avg_sq"]),
                           step=state["step"], step_factor=f, step_increment_bugfix=self.stepfix,
                           grad_scale=self.grad_scale)

    def _step_flat(self, f: torch.Tensor) -> None:
        rt = self._runtime
        group_of: Dict[int, Dict[str, Any]] = {}
        for group in self.param_groups:
            for p in group["params"]:
                group_of[id(p)] = group
        for slot in rt.slots:
            p = slot.param
            group = group_of.get(id(p))
            if group is None or not p.requires_grad:
                continue
            if slot.aware or rt.grad_shard is not None:
                g = rt.grad_view(slot)
            elif p.grad is not None:
                g = p.grad
            else:
                continue
            state = self.state[p]
            lowp = rt._own_rows_lowp(slot) if slot.aware and rt.lowp is not None and rt.lowp.dtype == torch.bfloat16 else None
            lr = group["lr"]
            if rt.symmetric and state["exp_avg"].dtype == torch.float32:
                # one kernel: AdamW on this rank's rows + bf16 stores into every peer's parameter buffer (the all-gather)
                step_in = state["step"] if self.stepfix else torch.zeros_like(state["step"])
                if rt.adamw_scatter(slot, state["exp_avg"], state["exp_avg_sq"], step_in,
                                    lr=float(lr) if not torch.is_tensor(lr) else float(lr.item()), betas=group["betas"],
                                    eps=group["eps"], weight_decay=group["weight_decay"], step_factor=f,
                                    grad_scale=self.grad_scale):
                    if self.stepfix:
                        state["step"].add_(f.to(state["step"].dtype))
                    continue
            adamw_step(p.data, g.reshape(p.shape), lr=float(lr) if not torch.is_tensor(lr) else float(lr.item()),
                       betas=group["betas"], eps=group["eps"], weight_decay=group["weight_decay"],
                       exp_avg=state["exp_avg"], exp_avg_sq=state["exp_avg_sq"], step=state["step"], step_factor=f,
                       step_increment_bugfix=self.stepfix, grad_scale=self.grad_scale,
                       lowp=lowp if lowp is not None and lowp.is_contiguous() else None)
            if slot.aware and rt.lowp is not None and (lowp is None or not lowp.is_contiguous()):
                rt._own_rows_lowp(slot).copy_(p.data)
        rt.all_gather_lowp(only_unfused=rt.symmetric)
        rt.finish_scatter()


@OptimConfig.register("adamw")
@dataclass
class AdamWConfig(OptimConfig[torch.optim.AdamW]):
    """
    Plain AdamW. It builds :class:`SkipStepAdamW` with skipping disabled (identical update rule), so that the
    same fused kernel and flat-buffer fast path are used; pass ``fused=False, foreach=False`` together with a
    model that is not managed by the sharded-parameter runtime to get ``torch.optim.AdamW`` itself.
    """

    lr: float = 1e-3
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-2
    foreach: Optional[bool] = None
    fused: Optional[bool] = None

    @classmethod
    def optimizer(cls) -> Type[torch.optim.AdamW]:
        return torch.optim.AdamW

    def build(self, model, strict: bool = True):
        if self.fused is False and self.foreach is False and getattr(model, "_sharding_runtime", None) is None:
            return super().build(model, strict=strict)
        cfg = SkipStepAdamWConfig(lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.weight_decay,
                                  group_overrides=self.group_overrides, compile=self.compile, fixed_fields=self.fixed_fields)
        optim = cfg.build(model, strict=strict)
        optim.skip_enabled = False
        # The param groups carry the fields torch.optim.AdamW groups have, so a checkpoint written here loads into an
        # optimizer that the reference builds from the same AdamWConfig (its loader wants every field of its groups).
        for group in optim.param_groups:
            for field, value in (("amsgrad", False), ("maximize", False), ("foreach", self.foreach), ("capturable", False),
                                 ("differentiable", False), ("fused", self.fused), ("decoupled_weight_decay", True)):
                group.setdefault(field, value)
        return optim


@OptimConfig.register("skip_step_adamw")
@dataclass
class SkipStepAdamWConfig(OptimConfig[SkipStepAdamW]):
    lr: float = 1e-3
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-2
    dtype: Optional[DType] = None
    foreach: bool = True
    step_increment_bugfix: bool = True
    rolling_interval_length: int = 128
    sigma_factor: int = 6

    @classmethod
    def optimizer(cls) -> Type[SkipStepAdamW]:
        return SkipStepAdamW
