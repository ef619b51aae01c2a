"""
Mixture-of-experts feed-forward layers (API of src/olmo_core/nn/moe/moe.py:58-426): router, optional
shared dense MLP, and the routed experts, combined as ``shared/(k+1) + routed*k/(k+1)``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple, Union

import torch
import torch.nn as nn

from ...config import DType, StrEnum
from ...exceptions import OLMoConfigurationError
from ...ops import attach_auxiliary_loss
from ..buffer_cache import BufferCache
from ..config import ModuleConfig
from ..feed_forward import FeedForwardConfig
from .loss import MoELoadBalancingLossGranularity
from .mlp import DroplessMoEMLP, MoEMLP
from .parallel_mlp import ParallelDroplessMLP, ParallelMLP, ParallelMLPBase
from .router import MoERouterConfig

__all__ = ["MoEBase", "MoE", "DroplessMoE", "MoEConfig", "MoEType"]


class MoEType(StrEnum):
    default = "default"
    dropless = "dropless"


@dataclass
class MoEConfig(ModuleConfig):
    name: MoEType = MoEType.default
    num_experts: int = 1
    hidden_size: int = 256
    capacity_factor: Optional[float] = None
    router: MoERouterConfig = field(default_factory=MoERouterConfig)
    shared_mlp: Optional[FeedForwardConfig] = None
    lb_loss_weight: Optional[float] = 0.01
    lb_loss_granularity: MoELoadBalancingLossGranularity = MoELoadBalancingLossGranularity.local_batch
    z_loss_weight: Optional[float] = None
    scale_loss_by_num_layers: bool = True
    dtype: DType = DType.float32

    def num_params(self, d_model: int) -> int:
        n = self.router.num_params(d_model, self.num_experts) + 3 * d_model * self.hidden_size * self.num_experts
        if self.shared_mlp is not None:
            n += self.shared_mlp.num_params(d_model)
        return n

    def num_active_params(self, d_model: int) -> int:
        return self.num_params(d_model) - 3 * d_model * self.hidden_size * (self.num_experts - self.router.top_k)

    def build(self, d_model: int, *, n_layers: int = 1, init_device: str = "cpu",
              cache: Optional[BufferCache] = None) -> "MoEBase":
        kwargs = self.as_dict(exclude_none=True, recurse=False)
        kwargs.pop("name")
        kwargs.update(d_model=d_model, n_layers=n_layers, init_device=init_device,
                      dtype=DType(kwargs.pop("dtype")).as_pt(), cache=cache)
        try:
            if self.name == MoEType.default:
                return MoE(**kwargs)
            if self.name == MoEType.dropless:
                return DroplessMoE(**kwargs)
            raise NotImplementedError(self.name)
        except TypeError as e:
            raise OLMoConfigurationError(f"invalid options for '{self.name}' {self.__class__.__name__}, {e}") from e


class MoEBase(nn.Module):
    def __init__(
        self,
        *,
        d_model: int,
        num_experts: int,
        hidden_size: int,
        router: MoERouterConfig,
        shared_mlp: Optional[FeedForwardConfig] = None,
        init_device: str = "cpu",
        lb_loss_weight: Optional[float] = None,
        lb_loss_granularity: MoELoadBalancingLossGranularity = MoELoadBalancingLossGranularity.local_batch,
        z_loss_weight: Optional[float] = None,
        n_layers: int = 1,
        scale_loss_by_num_layers: bool = True,
        dtype: torch.dtype = torch.float32,
        cache: Optional[BufferCache] = None,
        **kwargs,
    ):
        super().__init__()
        if scale_loss_by_num_layers:
            lb_loss_weight = None if lb_loss_weight is None else lb_loss_weight / n_layers
            z_loss_weight = None if z_loss_weight is None else z_loss_weight / n_layers
        self.router = router.build(d_model, num_experts, lb_loss_weight=lb_loss_weight,
                                   lb_loss_granularity=lb_loss_granularity, z_loss_weight=z_loss_weight, dtype=dtype,
                                   init_device=init_device)
        self.experts = self._init_parallel_mlp(d_model=d_model, num_experts=num_experts, hidden_size=hidden_size,
                                               dtype=dtype, init_device=init_device, cache=cache, **kwargs)
        self.shared_mlp = None if shared_mlp is None else shared_mlp.build(d_model, dtype=dtype, init_device=init_device)
        self._ep_enabled = False

    @property
    def num_experts(self) -> int:
        return self.router.num_experts

    @property
    def top_k(self) -> int:
        return self.router.top_k

    @property
    def ep_enabled(self) -> bool:
        return self._ep_enabled

    def warmup_cache(self, max_local_microbatch_size: int) -> None:
        if hasattr(self.experts, "warmup_cache"):
            self.experts.warmup_cache(max_local_microbatch_size)

    def compute_metrics(self, reset: bool = True) -> Dict[str, Tuple[torch.Tensor, Optional[object]]]:
        return self.router.compute_metrics(reset=reset)

    def reset_metrics(self) -> None:
        self.router.reset_metrics()

    def post_batch(self, dry_run: bool = False) -> None:
        self.router.post_batch(dry_run=dry_run)

    def _init_parallel_mlp(self, **kwargs) -> ParallelMLPBase:
        raise NotImplementedError

    def forward(self, x: torch.Tensor, *, loss_div_factor: Optional[Union[torch.Tensor, float]] = None) -> torch.Tensor:
        weights, indices, counts, aux = self.router(x, loss_div_factor=loss_div_factor)
        if aux is not None:
            x = attach_auxiliary_loss(x, aux)
        shared = self.shared_mlp(x) if self.shared_mlp is not None else None
        out = self.experts(x, weights, indices, counts)
        if shared is not None:
            k = self.top_k
            out = shared / (k + 1) + out * (k / (k + 1))
        return out

    def apply_pp(self, pp_mesh) -> None:
        from ...distributed.parallel import flatten_mesh, get_pp_stage_mesh, get_world_mesh

        world = get_world_mesh()
        assert world is not None
        self.router.group = flatten_mesh(get_pp_stage_mesh(world, pp_mesh)).get_group()

    def apply_ep(self, ep_mesh, **kwargs) -> None:
        self.experts.apply_ep(ep_mesh, **kwargs)
        self._ep_enabled = True

    def prepare_experts_for_fsdp(self, **kwargs) -> None:
        self.experts.prepare_experts_for_fsdp(**kwargs)

    def prepare_experts_for_ddp(self, **kwargs) -> None:
        self.experts.prepare_experts_for_ddp(**kwargs)

    def apply_cp(self, cp_mesh) -> None:
        self.router.apply_cp(cp_mesh)

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        self.router.apply_tp(tp_mesh)
        self.experts.apply_tp(tp_mesh)

    def num_flops_per_token(self, seq_len: int) -> int:
        n = 6 * sum(p.numel() for p in self.router.parameters())
        if self.shared_mlp is not None:
            n += self.shared_mlp.num_flops_per_token(seq_len)
        return n + self.experts.num_flops_per_token(seq_len)


class MoE(MoEBase):
    """Experts with a fixed capacity (tokens over capacity are dropped)."""

    def __init__(self, *, capacity_factor: float = 1.2, **kwargs):
        super().__init__(capacity_factor=capacity_factor, **kwargs)

    def _init_parallel_mlp(self, *, d_model, num_experts, hidden_size, dtype=torch.float32, init_device="cpu", cache=None,
                           capacity_factor: float = 1.2, **kwargs) -> ParallelMLPBase:
        return ParallelMLP(
            mlp=MoEMLP(d_model=d_model, hidden_size=hidden_size, num_experts=num_experts, dtype=dtype, init_device=init_device),
            top_k=self.router.top_k, capacity_factor=capacity_factor, cache=cache,
        )


class DroplessMoE(MoEBase):
    """Experts that process every routed token."""

    def _init_parallel_mlp(self, *, d_model, num_experts, hidden_size, dtype=torch.float32, init_device="cpu", cache=None,
                           **kwargs) -> ParallelMLPBase:
        return ParallelDroplessMLP(
            mlp=DroplessMoEMLP(d_model=d_model, hidden_size=hidden_size, num_experts=num_experts, dtype=dtype,
                               init_device=init_device),
            top_k=self.router.top_k, cache=cache,
        )
