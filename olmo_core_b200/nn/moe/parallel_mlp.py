"""
Orchestration of the expert computation, with and without expert parallelism
(role of src/olmo_core/nn/moe/parallel_mlp.py:34-871).

Single group of experts (no EP): sort routed copies by expert -> gather -> experts -> weighted scatter.
Expert parallel: each rank additionally exchanges its expert-sorted rows with the ranks that own the
experts (all-to-all with per-rank counts), runs its local experts, and sends results back.
"""

from __future__ import annotations

from typing import Any, List, NamedTuple, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ...distributed.utils import get_world_size
from ...ops import moe as ops
from .mlp import DroplessMoEMLP, MoEMLP, MoEMLPBase

__all__ = ["ParallelMLPBase", "ParallelMLP", "ParallelDroplessMLP", "PermutedAllToAllOutput"]


class PermutedAllToAllOutput(NamedTuple):
    """What a dispatch hands to the expert computation (field names of src/olmo_core/nn/moe/parallel_mlp.py:22-31)."""

    parallel_x: torch.Tensor
    parallel_indices: torch.Tensor
    parallel_bin_ids: Optional[torch.Tensor]
    parallel_bins: torch.Tensor
    parallel_batch_size_per_expert: torch.Tensor
    recv_counts: Optional[List[int]]
    send_counts: Optional[List[int]]
    expert_capacity: int
    handle: Any


class ParallelMLPBase(nn.Module):
    def __init__(self, *, mlp: MoEMLPBase, top_k: int, cache=None):
        super().__init__()
        self.mlp = mlp
        self.top_k = top_k
        self._ep_pg: Optional[dist.ProcessGroup] = None
        self._expert_parallel_enabled = False

    @property
    def d_model(self) -> int:
        return self.mlp.d_model

    @property
    def num_experts(self) -> int:
        return self.mlp.num_experts

    @property
    def num_local_experts(self) -> int:
        return self.mlp.num_local_experts

    @property
    def ep_world_size(self) -> int:
        return get_world_size(self._ep_pg) if self._ep_pg is not None else 1

    @property
    def ep_pg(self) -> Optional[dist.ProcessGroup]:
        return self._ep_pg

    def apply_ep(self, ep_mesh, **kwargs) -> None:
        self.mlp.apply_ep(ep_mesh, **kwargs)
        self._ep_pg = ep_mesh.get_group()
        self._expert_parallel_enabled = True

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        self.mlp.apply_tp(tp_mesh, **kwargs)
        self._ep_pg = tp_mesh.get_group()
        self._expert_parallel_enabled = True

    @property
    def hidden_sharding_degree(self) -> int:
        return self.mlp.hidden_sharding_degree

    def warmup_cache(self, max_local_microbatch_size: int) -> None:
        """Pre-size per-batch buffers; only the capacity-based variant keeps any."""
        del max_local_microbatch_size

    def prepare_experts_for_fsdp(self, **kwargs) -> None:
        """Expert weights are already partitioned by expert; data-parallel sharding treats them like any parameter."""
        self.mlp.prepare_experts_for_fsdp(**kwargs)

    def prepare_experts_for_ddp(self, **kwargs) -> None:
        self.mlp.prepare_experts_for_ddp(**kwargs)

    def indices_and_bins(self, expert_indices: torch.Tensor, batch_size_per_expert: torch.Tensor):
        return ops.indices_and_bins(expert_indices, self.num_experts, batch_size_per_expert)

    def forward(self, x: torch.Tensor, expert_weights: torch.Tensor, expert_indices: torch.Tensor,
                batch_size_per_expert: torch.Tensor) -> torch.Tensor:
        """``x``: ``[B, S, d]``; weights/indices ``[B, S, k]``; returns ``[B, S, d]``."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        w = expert_weights.reshape(-1, self.top_k)
        idx = expert_indices.reshape(-1, self.top_k)
        if self._expert_parallel_enabled and self.ep_world_size > 1:
            out = self.parallel_forward_once(x2, w, idx, batch_size_per_expert)
        else:
            out = self.forward_once(x2, w, idx, batch_size_per_expert)
        return out.view(shape)

    def forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        raise NotImplementedError

    def parallel_forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        raise NotImplementedError

    def num_flops_per_token(self, seq_len: int) -> int:
        per_expert = 3 * self.mlp.d_model * self.mlp.hidden_size
        return 6 * per_expert * self.top_k


class ParallelDroplessMLP(ParallelMLPBase):
    """Every routed copy is processed (no capacity limit)."""

    def __init__(self, *, mlp: DroplessMoEMLP, top_k: int, cache=None):
        super().__init__(mlp=mlp, top_k=top_k, cache=cache)

    def forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        indices, bin_ids, bins = self.indices_and_bins(expert_indices, batch_size_per_expert)
        xs = ops.gather(x, indices, bin_ids, bins, self.top_k)
        offsets = getattr(bins, "_offsets", None)  # set by the CUDA counting sort: the kernels read it on the device
        if offsets is not None and xs.is_cuda and xs.dtype == torch.bfloat16:
            offsets._is_offsets = True  # type: ignore[attr-defined]
            ys = self.mlp(xs, offsets)
        else:
            ys = self.mlp(xs, batch_size_per_expert.tolist())
        return ops.scatter(ys, indices, bin_ids, expert_weights, bins, self.top_k)

    def parallel_forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        ep, E_local = self.ep_world_size, self.num_local_experts
        indices, bin_ids, bins = self.indices_and_bins(expert_indices, batch_size_per_expert)
        from ...ops import moe_peer

        if indices.dtype == torch.int32 and moe_peer.peer_exchange_enabled(x, self._ep_pg):
            # permutation + transfer in one kernel over peer memory, both ways; rows arrive grouped by local expert
            ex = moe_peer.PeerExpertExchange.get(self._ep_pg, x.shape[1], indices.numel(), x.device)
            tables = ex.tables(batch_size_per_expert, E_local)
            recv = moe_peer.dispatch(x, indices, self.top_k, ex, tables)
            tables.offsets._is_offsets = True  # type: ignore[attr-defined]
            ys = self.mlp(recv, tables.offsets)
            back = moe_peer.combine(ys, indices.numel(), ex, tables)
            return ops.scatter(back, indices, bin_ids, expert_weights, bins, self.top_k)
        # Tokens per (destination rank, local expert) that we send, and that every peer sends us.
        send_counts = batch_size_per_expert.to(torch.int64).view(ep, E_local)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts.view(-1), send_counts.contiguous().view(-1), group=self._ep_pg)
        xs = ops.gather(x, indices, bin_ids, bins, self.top_k)
        send_list = send_counts.sum(dim=1).tolist()  # one host synchronisation for both split lists
        recv_mat = recv_counts.tolist()
        recv_list = [sum(r) for r in recv_mat]
        recv_x, _ = ops.all_to_all(xs, recv_list, send_list, group=self._ep_pg)
        # Received rows are ordered (source rank, local expert); regroup them by local expert.
        owner = torch.repeat_interleave(
            torch.arange(E_local, device=x.device).repeat(ep),
            torch.tensor([c for r in recv_mat for c in r], device=x.device),
            output_size=sum(recv_list),
        )
        order = torch.sort(owner, stable=True)[1]
        local_sizes = [sum(recv_mat[r][e] for r in range(ep)) for e in range(E_local)]
        ys_sorted = self.mlp(recv_x.index_select(0, order), local_sizes)
        ys = torch.empty_like(ys_sorted).index_copy(0, order, ys_sorted)
        back, _ = ops.all_to_all(ys, send_list, recv_list, group=self._ep_pg)
        return ops.scatter(back, indices, bin_ids, expert_weights, bins, self.top_k)


class ParallelMLP(ParallelMLPBase):
    """Fixed expert capacity: tokens beyond ``capacity`` per expert are dropped."""

    def __init__(self, *, mlp: MoEMLP, top_k: int, capacity_factor: float, cache=None, max_local_microbatch_size: Optional[int] = None):
        super().__init__(mlp=mlp, top_k=top_k, cache=cache)
        self.capacity_factor = capacity_factor
        self.max_local_microbatch_size = max_local_microbatch_size

    def expert_capacity(self, local_batch_size: int) -> int:
        n = local_batch_size if not self.training or self.max_local_microbatch_size is None else self.max_local_microbatch_size
        return max(1, int(self.capacity_factor * self.top_k * n / self.num_experts))

    def warmup_cache(self, max_local_microbatch_size: int) -> None:
        self.max_local_microbatch_size = max_local_microbatch_size

    def forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        indices, _, bins = self.indices_and_bins(expert_indices, batch_size_per_expert)
        cap = self.expert_capacity(x.shape[0])
        xb = ops.binned_gather(x, indices, bins, cap, self.top_k)
        yb = self.mlp(xb)
        return ops.binned_scatter(yb, indices, expert_weights, bins, self.top_k)

    def parallel_forward_once(self, x, expert_weights, expert_indices, batch_size_per_expert) -> torch.Tensor:
        ep, E_local = self.ep_world_size, self.num_local_experts
        indices, _, bins = self.indices_and_bins(expert_indices, batch_size_per_expert)
        cap = self.expert_capacity(x.shape[0])
        xb = ops.binned_gather(x, indices, bins, cap, self.top_k)  # [E, cap, d], E = ep * E_local
        d = xb.shape[-1]
        recv, _ = ops.all_to_all(xb.view(ep * E_local * cap, d), group=self._ep_pg)
        # [src rank, local expert, cap, d] -> [local expert, src rank * cap, d]
        recv = recv.view(ep, E_local, cap, d).transpose(0, 1).reshape(E_local, ep * cap, d)
        y = self.mlp(recv)
        y = y.view(E_local, ep, cap, d).transpose(0, 1).reshape(ep * E_local * cap, d)
        back, _ = ops.all_to_all(y, group=self._ep_pg)
        return ops.binned_scatter(back.view(ep * E_local, cap, d), indices, expert_weights, bins, self.top_k)
