"""Mixture-of-experts building blocks (src/olmo_core/nn/moe/__init__.py:16-29)."""

from .loss import MoELoadBalancingLossGranularity
from .mlp import DroplessMoEMLP, MoEMLP
from .moe import DroplessMoE, MoE, MoEBase, MoEConfig, MoEType
from .router import MoELinearRouter, MoERouter, MoERouterConfig, MoERouterGatingFunction, MoERouterType

__all__ = [
    "DroplessMoE", "DroplessMoEMLP", "MoE", "MoEBase", "MoEConfig", "MoELinearRouter",
    "MoELoadBalancingLossGranularity", "MoEMLP", "MoERouter", "MoERouterConfig", "MoERouterGatingFunction",
    "MoERouterType", "MoEType",
]
