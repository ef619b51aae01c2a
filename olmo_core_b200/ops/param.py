"""
Access to parameters that are managed by the sharded-parameter runtime.

Such a parameter's ``.data`` holds only this rank's rows (fp32 master copy); the full compute copy is the
attribute ``_lowp`` and gradients are accumulated into the attribute ``main_grad`` (both views into flat
buffers). CUDA kernels read/write those buffers directly. Every other code path -- the PyTorch
reference math on CPU, fp32 debugging runs -- goes through :func:`full_param`, which returns the full
tensor as an autograd leaf-like value whose gradient is routed into ``main_grad``.
"""

from __future__ import annotations

from typing import Optional

import torch

__all__ = ["full_param", "is_managed"]


def is_managed(weight: torch.Tensor) -> bool:
    return getattr(weight, "_lowp", None) is not None


class _FullParam(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight: torch.Tensor, dtype: Optional[torch.dtype]):  # type: ignore[override]
        ctx.weight_ref = weight
        full = weight._lowp  # type: ignore[attr-defined]
        if dtype is not None and full.dtype != dtype:
            return full.to(dtype)
        return full.detach().view_as(full)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        weight = ctx.weight_ref
        weight.main_grad.add_(grad.to(weight.main_grad.dtype))  # type: ignore[attr-defined]
        return None, None


def full_param(weight: Optional[torch.Tensor], dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """The full tensor of ``weight`` (cast to ``dtype`` when given), differentiable for managed and plain parameters."""
    if weight is None:
        return None
    if not is_managed(weight):
        return weight if dtype is None or weight.dtype == dtype else weight.to(dtype)
    if not (weight.requires_grad and torch.is_grad_enabled()):
        full = weight._lowp  # type: ignore[attr-defined]
        return full if dtype is None or full.dtype == dtype else full.to(dtype)
    return _FullParam.apply(weight, dtype)
