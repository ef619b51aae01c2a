"""
Cross-entropy with optional z-loss (API of src/olmo_core/nn/functional/cross_entropy_loss.py:12-124).
Both functions dispatch to the CUDA kernels in ``olmo_core_b200.ops.loss`` for CUDA tensors and to the
PyTorch statement of the same formulas otherwise.
"""

from __future__ import annotations

from typing import Literal, Optional, Tuple

import torch

from ...ops.loss import cross_entropy_with_z_loss, fused_linear_cross_entropy

__all__ = ["cross_entropy_loss", "fused_linear_cross_entropy_loss"]


def cross_entropy_loss(
    logits: torch.Tensor,
    labels: torch.Tensor,
    *,
    ignore_index: int = -100,
    reduction: Literal["mean", "sum", "none"] = "mean",
    compute_z_loss: bool = False,
    z_loss_multiplier: float = 1e-4,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """
    ``logits``: ``(N, V)``, ``labels``: ``(N,)``. Returns ``(ce_loss, z_loss)``; the z-loss is
    ``z_loss_multiplier * logsumexp(logits)^2`` over non-ignored tokens, reduced like the CE term.
    """
    return cross_entropy_with_z_loss(logits, labels, ignore_index=ignore_index, reduction=reduction,
                                     compute_z_loss=compute_z_loss, z_loss_multiplier=z_loss_multiplier)


def fused_linear_cross_entropy_loss(
    _input: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    ce_weight: Optional[torch.Tensor] = None,
    ignore_index: int = -100,
    reduction: Literal["mean", "sum", "none"] = "mean",
    label_smoothing: float = 0.0,
    compute_z_loss: bool = False,
    z_loss_multiplier: float = 1e-4,
    softcap: Optional[float] = None,
    accum_dtype: Optional[torch.dtype] = None,
    loss_scale: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """
    Loss of ``_input @ weight.T`` against ``labels`` without materialising the logits. Returns
    ``(total loss = ce + z, z_loss)`` like the reference. ``loss_scale`` (a scalar tensor, e.g.
    ``1/loss_div_factor``) is folded into the gradients produced during the forward pass. Class weights
    (``ce_weight``), ``label_smoothing`` and ``softcap`` (logits squashed to ``softcap * tanh(logits / softcap)``) take
    the materialised PyTorch form.
    """
    del accum_dtype  # gradients are accumulated in fp32 always
    if ce_weight is not None or label_smoothing != 0.0 or softcap is not None:
        # class weights, label smoothing and logit soft-capping: the materialised form in plain PyTorch
        logits = torch.nn.functional.linear(_input, weight.to(_input.dtype), None if bias is None else bias.to(_input.dtype))
        lf = logits.float()
        if softcap is not None:
            lf = softcap * torch.tanh(lf / softcap)
        ce = torch.nn.functional.cross_entropy(lf, labels, weight=ce_weight, ignore_index=ignore_index, reduction=reduction,
                                               label_smoothing=label_smoothing)
        z = None
        if compute_z_loss:
            keep = (labels != ignore_index).to(lf.dtype)
            z = z_loss_multiplier * torch.logsumexp(lf, dim=-1).pow(2) * keep
            if reduction == "mean":
                z = z.sum() / keep.sum().clamp(min=1)
            elif reduction == "sum":
                z = z.sum()
        if loss_scale is not None:
            ce = ce * loss_scale
            z = z * loss_scale if z is not None else None
        return (ce + z if z is not None else ce), z
    if bias is not None or reduction == "none":
        logits = torch.nn.functional.linear(_input, weight.to(_input.dtype), None if bias is None else bias.to(_input.dtype))
        ce, z = cross_entropy_with_z_loss(logits, labels, ignore_index=ignore_index, reduction=reduction,
                                          compute_z_loss=compute_z_loss, z_loss_multiplier=z_loss_multiplier)
        if loss_scale is not None:
            ce = ce * loss_scale
            z = z * loss_scale if z is not None else None
        return (ce + z if z is not None else ce), z
    scale = loss_scale
    if reduction == "mean":
        denom = (labels != ignore_index).sum().clamp(min=1).to(torch.float32)
        scale = (1.0 / denom) if scale is None else scale / denom
    ce, z = fused_linear_cross_entropy(_input, weight, labels, ignore_index=ignore_index,
                                       z_loss_multiplier=z_loss_multiplier if compute_z_loss else None, scale=scale)
    return (ce + z if z is not None else ce), z
