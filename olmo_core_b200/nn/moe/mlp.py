"""
Expert MLP weights and the grouped expert computation (API of src/olmo_core/nn/moe/mlp.py:32-293).

Weights of all (local) experts live in single parameters whose first two dimensions are flattened so
that data-parallel sharding can split dim 0: ``DroplessMoEMLP`` stores ``w1, w2, w3`` as
``[E * hidden, d_model]``; ``MoEMLP`` (fixed capacity, batched matmul) stores ``w1, w3`` as
``[E * d_model, hidden]`` and ``w2`` as ``[E * hidden, d_model]``.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...distributed.utils import get_local_tensor
from ...exceptions import OLMoConfigurationError
from ...ops.elementwise import swiglu
from ...ops.gemm import LinearFunction, gemm

__all__ = ["MoEMLPBase", "MoEMLP", "DroplessMoEMLP"]


class MoEMLPBase(nn.Module):
    def __init__(self, *, d_model: int, hidden_size: int, num_experts: int):
        super().__init__()
        self.d_model = d_model
        self.hidden_size = hidden_size
        self.num_experts = num_experts
        self.num_local_experts = num_experts
        self.hidden_sharding_degree = 1
        self.ep_mesh = None
        self.ep_pg = None

    def _shard_experts(self, ep_mesh) -> None:
        """Keep only this rank's contiguous block of experts (dim-0 sharding of every weight)."""
        pg = ep_mesh.get_group()
        import torch.distributed as dist

        ws, rank = dist.get_world_size(pg), dist.get_rank(pg)
        if self.num_experts % ws != 0:
            raise OLMoConfigurationError(f"'num_experts' ({self.num_experts}) must be divisible by the expert parallel degree ({ws})")
        self.ep_mesh, self.ep_pg = ep_mesh, pg
        self.num_local_experts = self.num_experts // ws
        for name in ("w1", "w2", "w3"):
            p = getattr(self, name)
            rows = p.shape[0] // ws
            if p.device.type == "meta":
                local = torch.empty((rows,) + tuple(p.shape[1:]), dtype=p.dtype, device="meta")
            else:
                local = p.data.narrow(0, rank * rows, rows).clone()
            new = nn.Parameter(local, requires_grad=p.requires_grad)
            new._ep_shard = (rank, ws)  # type: ignore[attr-defined]
            setattr(self, name, new)

    def apply_ep(self, ep_mesh, **kwargs) -> None:
        self._shard_experts(ep_mesh)

    def apply_tp(self, tp_mesh, **kwargs) -> None:
        """Tensor parallelism for MoE = expert sharding over the TP group."""
        self._shard_experts(tp_mesh)

    def prepare_experts_for_fsdp(self, *, world_mesh=None, **kwargs) -> None:
        """
        Called before the model is sharded for data parallelism (src/olmo_core/nn/moe/mlp.py:87-112). The local
        expert block is an ordinary parameter here (marked with its expert-parallel rank), and the data-parallel
        runtime partitions it over the ranks that hold the same block, so there is nothing to re-wrap.
        """
        del world_mesh, kwargs

    def prepare_experts_for_ddp(self, *, world_mesh=None) -> None:
        del world_mesh


class MoEMLP(MoEMLPBase):
    """Capacity-based experts: ``x`` is ``[E_local, capacity, d]`` and each expert is a batched matmul."""

    def __init__(self, *, d_model: int, hidden_size: int, num_experts: int, dtype: torch.dtype = torch.float32,
                 init_device: str = "cpu"):
        super().__init__(d_model=d_model, hidden_size=hidden_size, num_experts=num_experts)
        self.w1 = nn.Parameter(torch.empty(num_experts * d_model, hidden_size, device=init_device, dtype=dtype))
        self.w2 = nn.Parameter(torch.empty(num_experts * hidden_size, d_model, device=init_device, dtype=dtype))
        self.w3 = nn.Parameter(torch.empty(num_experts * d_model, hidden_size, device=init_device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for w in (self.w1, self.w2, self.w3):
            if w.device.type != "meta":
                nn.init.trunc_normal_(w, std=0.02, a=-0.06, b=0.06)

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.d_model}, hidden_size={self.hidden_size}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        E = self.num_local_experts
        w1 = get_local_tensor(self.w1).view(E, self.d_model, self.hidden_size).to(x.dtype)
        w2 = get_local_tensor(self.w2).view(E, self.hidden_size, self.d_model).to(x.dtype)
        w3 = get_local_tensor(self.w3).view(E, self.d_model, self.hidden_size).to(x.dtype)
        return torch.bmm(F.silu(torch.bmm(x, w1)) * torch.bmm(x, w3), w2)


class _GroupedLinear(torch.autograd.Function):
    """
    ``y[rows of expert e] = x[rows of expert e] @ w_e^T`` (``trans_b``) or ``@ w_e``, for expert-sorted rows.
    Forward, dgrad and wgrad are ONE grouped tcgen05 GEMM launch each; the group boundaries are a device tensor
    (``offsets``, int32 ``[E + 1]``), so the host never waits for the routing result. The weight gradient accumulates into
    ``weight.main_grad`` when the sharded-parameter runtime provides one.
    """

    @staticmethod
    def forward(ctx, x, weight, offsets, trans_b: bool):  # type: ignore[override]
        from ...ops.gemm import compute_weight, grouped_gemm

        w = compute_weight(weight, torch.bfloat16)
        x = x.contiguous()
        y = grouped_gemm(x, w, offsets, trans_b=trans_b)
        ctx.save_for_backward(x, w, offsets)
        ctx.trans_b, ctx.weight_ref = trans_b, weight
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        from ...ops.gemm import grouped_gemm, grouped_gemm_wgrad

        x, w, offsets = ctx.saved_tensors
        trans_b, weight = ctx.trans_b, ctx.weight_ref
        dy = dy.contiguous()
        # y = x w^T: dx = dy w, dw = dy^T x.   y = x w: dx = dy w^T, dw = x^T dy.
        dx = grouped_gemm(dy, w, offsets, trans_b=not trans_b)
        main_grad = getattr(weight, "main_grad", None)
        dw = main_grad if main_grad is not None else torch.empty(w.shape, dtype=torch.float32, device=x.device)
        a, b = (dy, x) if trans_b else (x, dy)
        grouped_gemm_wgrad(a, b, offsets, dw.view(w.shape), accumulate=main_grad is not None)
        if main_grad is not None:
            return dx, None, None, None
        return dx, dw.to(weight.dtype), None, None


class DroplessMoEMLP(MoEMLPBase):
    """Dropless experts: rows sorted by expert with a variable number of rows per expert."""

    def __init__(self, *, d_model: int, hidden_size: int, num_experts: int, dtype: torch.dtype = torch.float32,
                 init_device: str = "cpu"):
        super().__init__(d_model=d_model, hidden_size=hidden_size, num_experts=num_experts)
        self.w1 = nn.Parameter(torch.empty(num_experts * hidden_size, d_model, device=init_device, dtype=dtype))
        self.w2 = nn.Parameter(torch.empty(num_experts * hidden_size, d_model, device=init_device, dtype=dtype))
        self.w3 = nn.Parameter(torch.empty(num_experts * hidden_size, d_model, device=init_device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for w in (self.w1, self.w2, self.w3):
            if w.device.type != "meta":
                nn.init.trunc_normal_(w, std=0.02, a=-0.06, b=0.06)

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.d_model}, hidden_size={self.hidden_size}"

    def gmm(self, x: torch.Tensor, w: torch.Tensor, batch_sizes, trans_b: bool = False) -> torch.Tensor:
        """
        Grouped matmul over expert-sorted rows. ``w``: ``[E_local * hidden, d_model]``. ``batch_sizes``: rows per expert,
        a list or a tensor; on the kernel path a device tensor is consumed as is (no host synchronisation).
        """
        E = self.num_local_experts
        if x.is_cuda and x.dtype == torch.bfloat16:
            return _GroupedLinear.apply(x, w, self._offsets(batch_sizes, x.device), trans_b)
        if torch.is_tensor(batch_sizes):
            batch_sizes = batch_sizes.tolist()
        from ...ops.param import full_param

        wv = full_param(w, x.dtype).view(E, self.hidden_size, self.d_model)
        outs = []
        r = 0
        for e, n in enumerate(batch_sizes):
            xs = x[r:r + n]
            outs.append(xs @ wv[e].t() if trans_b else xs @ wv[e])
            r += n
        return torch.cat(outs, dim=0) if outs else x.new_zeros((0, wv.shape[1] if trans_b else wv.shape[2]))

    @staticmethod
    def _offsets(batch_sizes, device) -> torch.Tensor:
        """Row prefix sums ``[E + 1]`` (int32, on ``device``) from rows per expert; a ready ``[E + 1]`` tensor passes through."""
        if torch.is_tensor(batch_sizes) and getattr(batch_sizes, "_is_offsets", False):
            return batch_sizes
        sizes = batch_sizes if torch.is_tensor(batch_sizes) else torch.tensor(list(batch_sizes), dtype=torch.int32)
        sizes = sizes.to(device=device, dtype=torch.int32, non_blocking=True)
        offsets = torch.zeros(sizes.numel() + 1, dtype=torch.int32, device=device)
        torch.cumsum(sizes, 0, out=offsets[1:])
        offsets._is_offsets = True  # type: ignore[attr-defined]
        return offsets

    def forward(self, x: torch.Tensor, batch_size_per_expert) -> torch.Tensor:
        """``x``: ``[rows, d]`` sorted by local expert; ``batch_size_per_expert``: list or tensor of row counts."""
        sizes = batch_size_per_expert
        if x.is_cuda and x.dtype == torch.bfloat16:
            sizes = self._offsets(batch_size_per_expert, x.device)  # computed once, shared by the three products
        w1, w2, w3 = (get_local_tensor(w) for w in (self.w1, self.w2, self.w3))
        a = self.gmm(x, w1, sizes, trans_b=True)
        b = self.gmm(x, w3, sizes, trans_b=True)
        return self.gmm(swiglu(a, b), w2, sizes, trans_b=False)
