"""
MoE routers (API of src/olmo_core/nn/moe/router.py:49-572): fp32 logits, softmax or sigmoid gating,
top-k selection (optionally with the DeepSeek-v3 auxiliary-loss-free score bias), optional weight
renormalisation, per-expert token counts and the auxiliary losses.
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ...config import DType, StrEnum
from ...distributed.utils import get_local_tensor, is_distributed
from ...exceptions import OLMoConfigurationError
from ...ops import moe as moe_ops
from ..config import ModuleConfig
from .loss import MoELoadBalancingLossGranularity, load_balancing_loss, router_z_loss

__all__ = ["MoERouter", "MoELinearRouter", "MoERouterConfig", "MoERouterType", "MoERouterGatingFunction"]


class MoERouterType(StrEnum):
    default = "default"


class MoERouterGatingFunction(StrEnum):
    softmax = "softmax"
    sigmoid = "sigmoid"


@dataclass
class MoERouterConfig(ModuleConfig):
    name: MoERouterType = MoERouterType.default
    top_k: int = 1
    jitter_eps: Optional[float] = None
    normalize_expert_weights: Optional[float] = None
    uniform_expert_assignment: bool = False
    bias_gamma: Optional[float] = None
    gating_function: MoERouterGatingFunction = MoERouterGatingFunction.softmax
    dtype: Optional[DType] = None

    def num_params(self, d_model: int, num_experts: int) -> int:
        if self.name != MoERouterType.default:
            raise NotImplementedError(self.name)
        return d_model * num_experts

    def build(self, d_model: int, num_experts: int, *, lb_loss_weight: Optional[float] = None,
              lb_loss_granularity: MoELoadBalancingLossGranularity = MoELoadBalancingLossGranularity.local_batch,
              z_loss_weight: Optional[float] = None, dtype: Optional[torch.dtype] = None,
              init_device: str = "cpu") -> "MoERouter":
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        kwargs.update(d_model=d_model, num_experts=num_experts, init_device=init_device, lb_loss_weight=lb_loss_weight,
                      lb_loss_granularity=lb_loss_granularity, z_loss_weight=z_loss_weight)
        if self.dtype is not None:
            kwargs["dtype"] = self.dtype.as_pt()
        elif dtype is not None:
            kwargs["dtype"] = dtype
        try:
            return MoELinearRouter(**kwargs)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


class _FusedSoftmaxTopK(torch.autograd.Function):
    """
    ``logits [N, E] -> (softmax scores [N, E], top-k weights [N, k], expert ids [N, k], tokens per expert [E])`` in one
    kernel (one warp per token keeps its row in registers). Backward is the softmax Jacobian applied to the sum of the
    gradients that arrive through the scores (auxiliary loss) and through the selected weights.
    """

    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int):  # type: ignore[override]
        from ...ops import _lib

        n, e = logits.shape
        scores = torch.empty((n, e), dtype=torch.float32, device=logits.device)
        weights = torch.empty((n, top_k), dtype=torch.float32, device=logits.device)
        experts = torch.empty((n, top_k), dtype=torch.int32, device=logits.device)
        counts = torch.empty(e, dtype=torch.int32, device=logits.device)
        rc = _lib.lib().ocb_moe_router_topk(logits.data_ptr(), scores.data_ptr(), weights.data_ptr(), experts.data_ptr(),
                                            counts.data_ptr(), n, e, top_k, 0, 0, logits.stride(0), _lib.dt(logits),
                                            _lib.stream_ptr())
        _lib.check(rc, "ocb_moe_router_topk")
        ids = experts.long()
        ctx.save_for_backward(scores, ids)
        ctx.mark_non_differentiable(ids, counts)
        ctx.in_dtype = logits.dtype
        return scores, weights, ids, counts

    @staticmethod
    def backward(ctx, d_scores, d_weights, _ids, _counts):  # type: ignore[override]
        scores, ids = ctx.saved_tensors
        g = torch.zeros_like(scores) if d_scores is None else d_scores.float().clone()
        if d_weights is not None:
            g.scatter_add_(1, ids, d_weights.float())
        d_logits = scores * (g - (g * scores).sum(dim=-1, keepdim=True))
        return d_logits.to(ctx.in_dtype), None


class MoERouter(nn.Module):
    def __init__(
        self,
        *,
        d_model: int,
        num_experts: int,
        top_k: int = 1,
        jitter_eps: Optional[float] = None,
        normalize_expert_weights: Optional[float] = None,
        uniform_expert_assignment: bool = False,
        bias_gamma: Optional[float] = None,
        gating_function: MoERouterGatingFunction = MoERouterGatingFunction.softmax,
        lb_loss_weight: Optional[float] = None,
        lb_loss_granularity: MoELoadBalancingLossGranularity = MoELoadBalancingLossGranularity.local_batch,
        z_loss_weight: Optional[float] = None,
        init_device: str = "cpu",
    ):
        super().__init__()
        self.d_model = d_model
        self.num_experts = num_experts
        self.top_k = top_k
        self.jitter_eps = jitter_eps
        self.normalize_expert_weights = normalize_expert_weights
        self.uniform_expert_assignment = uniform_expert_assignment
        self.bias_gamma = bias_gamma
        self.gating_function = MoERouterGatingFunction(gating_function)
        self.lb_loss_weight = lb_loss_weight
        self.lb_loss_granularity = lb_loss_granularity
        self.z_loss_weight = z_loss_weight
        self.group: Optional[dist.ProcessGroup] = None
        self.cp_mesh = None
        self.tp_mesh = None
        if bias_gamma is not None:
            if bias_gamma <= 0:
                raise OLMoConfigurationError("'bias_gamma' must be positive")
            self.register_buffer("score_bias", torch.zeros(num_experts, device=init_device))
        else:
            self.register_buffer("score_bias", None)
        # Metric accumulators are plain attributes (a dict) so that parameter sharding, ``.to()`` and
        # ``state_dict()`` leave them alone; they are created lazily on the device of the inputs.
        self._acc: Dict[str, torch.Tensor] = {}

    def _accumulate(self, name: str, value: torch.Tensor) -> None:
        cur = self._acc.get(name)
        if cur is None or cur.device != value.device:
            self._acc[name] = value.detach().clone().float()
        else:
            cur += value.detach()

    @property
    def device(self) -> torch.device:
        """Device the metric accumulators live on (src/olmo_core/nn/moe/router.py:238-240)."""
        from ...utils import get_default_device

        return get_default_device()

    @property
    def batch_size_per_expert(self) -> Optional[torch.Tensor]:
        return self._acc.get("counts")

    @property
    def score_bias_batch_size_per_expert(self) -> Optional[torch.Tensor]:
        """Tokens per expert since the last score-bias update; ``None`` without auxiliary-loss-free balancing
        (src/olmo_core/nn/moe/router.py:242-261)."""
        if self.bias_gamma is None:
            return None
        return self._acc.get("bias_counts")

    @score_bias_batch_size_per_expert.setter
    def score_bias_batch_size_per_expert(self, value: torch.Tensor) -> None:
        self._acc["bias_counts"] = value

    @property
    def load_balancing_loss(self) -> Optional[torch.Tensor]:
        return self._acc.get("lb")

    @property
    def z_loss(self) -> Optional[torch.Tensor]:
        return self._acc.get("z")

    def reset_parameters(self) -> None:
        self._acc.clear()
        if self.score_bias is not None and self.score_bias.device.type != "meta":
            self.score_bias.zero_()

    @torch.no_grad()
    def post_batch(self, dry_run: bool = False) -> None:
        """Auxiliary-loss-free balancing: nudge each expert's score bias towards the mean load."""
        if self.bias_gamma is None or not self.training:
            return
        counts = self._acc.get("bias_counts")
        if counts is None:
            return
        if is_distributed():
            dist.all_reduce(counts, group=self.group)
        delta = self.bias_gamma * (counts.mean(dim=0, keepdim=True, dtype=torch.float32) - counts).sign()
        if not dry_run:
            get_local_tensor(self.score_bias).add_(delta.to(self.score_bias.dtype))
        counts.zero_()

    def jitter(self, x: torch.Tensor) -> torch.Tensor:
        if self.jitter_eps is None or not self.training:
            return x
        lo, hi = 1.0 - self.jitter_eps, 1.0 + self.jitter_eps
        return x * (lo + torch.rand_like(x) * (hi - lo))

    def get_top_k(self, scores: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.bias_gamma is None:
            if self.top_k == 1:
                weights, indices = scores.max(dim=-1, keepdim=True)
            else:
                weights, indices = torch.topk(scores, self.top_k, dim=-1)
        else:
            with torch.no_grad():
                _, indices = torch.topk(scores + self.score_bias.unsqueeze(0), self.top_k, dim=-1)
            weights = scores.gather(-1, indices)
        if self.uniform_expert_assignment:
            with torch.no_grad():
                indices = torch.remainder(torch.arange(indices.numel(), device=indices.device), self.num_experts).view_as(indices)
            weights = scores.gather(-1, indices)
        return weights, indices

    @abstractmethod
    def get_expert_logits(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    @torch.no_grad()
    def compute_metrics(self, reset: bool = True) -> Dict[str, Tuple[torch.Tensor, Optional[object]]]:
        from ...train.common import ReduceType

        out: Dict[str, Tuple[torch.Tensor, Optional[object]]] = {}
        counts = self._acc.get("counts")
        if counts is not None:
            out["load imbalance"] = (counts.max() / counts.mean(dtype=torch.float).clamp(min=1e-9), ReduceType.max)
        if self.lb_loss_weight is not None and "lb" in self._acc:
            out["load balancing loss"] = (self.lb_loss_weight * self._acc["lb"], ReduceType.mean)
            out["load balancing loss unscaled"] = (self._acc["lb"].clone(), ReduceType.mean)
        if self.z_loss_weight is not None and "z" in self._acc:
            out["router Z loss"] = (self.z_loss_weight * self._acc["z"], ReduceType.mean)
            out["router Z loss unscaled"] = (self._acc["z"].clone(), ReduceType.mean)
        if reset:
            self.reset_metrics()
        return out

    def reset_metrics(self) -> None:
        for k in ("counts", "lb", "z"):
            if k in self._acc:
                self._acc[k].zero_()

    def forward(self, x: torch.Tensor, *, loss_div_factor: Optional[Union[torch.Tensor, float]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
        """
        ``x``: ``[B, S, d]``. Returns weights ``[B, S, k]``, expert ids ``[B, S, k]``, tokens per expert
        ``[E]`` and the weighted auxiliary loss (or None).
        """
        x = self.jitter(x)
        logits = self.get_expert_logits(x).float()
        fused = (logits.is_cuda and self.gating_function == MoERouterGatingFunction.softmax and self.bias_gamma is None
                 and not self.uniform_expert_assignment and self.num_experts <= 1024 and self.top_k <= 32)
        if fused:
            flat = logits.reshape(-1, self.num_experts)
            scores, weights, indices, kernel_counts = _FusedSoftmaxTopK.apply(flat, self.top_k)
            scores = scores.view_as(logits)
            weights = weights.view(*logits.shape[:-1], self.top_k)
            indices = indices.view(*logits.shape[:-1], self.top_k)
        elif self.gating_function == MoERouterGatingFunction.softmax:
            scores = logits.softmax(dim=-1)
            weights, indices = self.get_top_k(scores)
        else:
            scores = torch.sigmoid(logits) + 1e-7
            weights, indices = self.get_top_k(scores)
        if self.normalize_expert_weights is not None:
            weights = weights / torch.norm(weights, p=self.normalize_expert_weights, dim=-1, keepdim=True)
        with torch.no_grad():
            if fused and self.lb_loss_granularity != MoELoadBalancingLossGranularity.instance:
                counts = kernel_counts.long()
                per_seq = counts.unsqueeze(0)  # only the per-instance loss reads the per-sequence histogram
            else:
                per_seq = moe_ops.batched_histc(indices, self.num_experts).sum(dim=1)  # [B, E]
                counts = per_seq.sum(dim=0)
        aux: Optional[torch.Tensor] = None
        if self.training and torch.is_grad_enabled():
            with torch.autocast(enabled=False, device_type=x.device.type):
                if self.lb_loss_weight is not None:
                    s = scores / scores.sum(dim=-1, keepdim=True) if self.gating_function == MoERouterGatingFunction.sigmoid else scores
                    lb = load_balancing_loss(
                        num_experts=self.num_experts, top_k=self.top_k, expert_scores=s, batch_size_per_expert=counts,
                        batched_batch_size_per_expert=per_seq, granularity=self.lb_loss_granularity,
                        loss_div_factor=loss_div_factor, tp_mesh=self.tp_mesh, cp_mesh=self.cp_mesh,
                    )
                    self._accumulate("lb", lb)
                    aux = self.lb_loss_weight * lb
                if self.z_loss_weight is not None:
                    z = router_z_loss(expert_logits=logits, loss_div_factor=loss_div_factor, tp_mesh=self.tp_mesh,
                                      cp_mesh=self.cp_mesh)
                    self._accumulate("z", z)
                    aux = self.z_loss_weight * z if aux is None else aux + self.z_loss_weight * z
            self._accumulate("counts", counts)
            if self.bias_gamma is not None:
                self._accumulate("bias_counts", counts)
        return weights, indices, counts, aux

    def apply_tp(self, tp_mesh, float8_enabled: bool = False) -> None:
        self.tp_mesh = tp_mesh

    def apply_cp(self, cp_mesh) -> None:
        self.cp_mesh = cp_mesh


class MoELinearRouter(MoERouter):
    """Learned linear router. The weight is stored flat ``[E * d]`` so that it shards over any world size."""

    def __init__(self, *, dtype: torch.dtype = torch.float32, init_device: str = "cpu", **kwargs):
        super().__init__(init_device=init_device, **kwargs)
        self.weight = nn.Parameter(torch.empty(self.num_experts * self.d_model, device=init_device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        super().reset_parameters()
        if self.weight.device.type != "meta":
            nn.init.trunc_normal_(self.weight, std=0.02, a=-0.06, b=0.06)

    def extra_repr(self) -> str:
        return f"in_features={self.d_model}, num_experts={self.num_experts}"

    def get_expert_logits(self, x: torch.Tensor) -> torch.Tensor:
        w = get_local_tensor(self.weight).view(self.num_experts, self.d_model)
        return F.linear(x.float(), w.float())
