"""Auxiliary MoE losses (src/olmo_core/nn/moe/loss.py:11-138)."""

from __future__ import annotations

from typing import Optional, Union

import torch
import torch.distributed as dist

from ...config import StrEnum

__all__ = ["MoELoadBalancingLossGranularity", "load_balancing_loss", "router_z_loss"]


class MoELoadBalancingLossGranularity(StrEnum):
    local_batch = "local_batch"
    """Computed over the rank-local tokens, whatever the parallelism."""
    instance = "instance"
    """Computed per sequence, with counts summed over context/tensor-parallel ranks."""


def _group_size(mesh) -> int:
    return 1 if mesh is None else mesh.size()


def load_balancing_loss(
    *,
    num_experts: int,
    top_k: int,
    expert_scores: torch.Tensor,
    batch_size_per_expert: torch.Tensor,
    batched_batch_size_per_expert: torch.Tensor,
    granularity: MoELoadBalancingLossGranularity,
    loss_div_factor: Optional[Union[torch.Tensor, float]] = None,
    tp_mesh=None,
    cp_mesh=None,
) -> torch.Tensor:
    """``(E / k) * sum_e count_e * mean_tokens(score_e) / div`` (Switch-style)."""
    B, S, _ = expert_scores.shape
    if granularity == MoELoadBalancingLossGranularity.instance:
        counts = batched_batch_size_per_expert.to(expert_scores.dtype)
        for mesh in (cp_mesh, tp_mesh):
            if mesh is not None:
                dist.all_reduce(counts, group=mesh.get_group())
        mean_scores = expert_scores.view(B, -1, num_experts).mean(dim=1)
        if tp_mesh is not None:
            ms = mean_scores.clone()
            dist.all_reduce(ms, group=tp_mesh.get_group())
            mean_scores = mean_scores + (ms / tp_mesh.size() - mean_scores).detach()
        div = loss_div_factor if loss_div_factor is not None else counts.sum() / top_k
        loss = (mean_scores * counts).sum() / div
    else:
        if loss_div_factor is None:
            div = B * S * _group_size(tp_mesh)
        else:
            div = loss_div_factor / _group_size(cp_mesh) if cp_mesh is not None else loss_div_factor
        counts = batch_size_per_expert.to(expert_scores.dtype)
        loss = torch.dot(counts, expert_scores.view(-1, num_experts).mean(dim=0)) / div
    return (num_experts / top_k) * loss


def router_z_loss(
    *,
    expert_logits: torch.Tensor,
    loss_div_factor: Optional[Union[torch.Tensor, float]] = None,
    tp_mesh=None,
    cp_mesh=None,
) -> torch.Tensor:
    """``sum logsumexp(logits)^2 / div``"""
    B, S, _ = expert_logits.shape
    if loss_div_factor is None:
        div = B * S * _group_size(tp_mesh)
    else:
        div = loss_div_factor / _group_size(cp_mesh) if cp_mesh is not None else loss_div_factor
    return torch.logsumexp(expert_logits, dim=-1).square().sum() / div
