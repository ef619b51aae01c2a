"""
Operator layer. Each op runs a hand-written sm_100a kernel (``csrc/*.cu``, bound through ctypes in
``_lib``) when its inputs live on a CUDA device and a PyTorch restatement of the same math otherwise.
"""

import torch

__all__ = ["attach_auxiliary_loss", "AutoAuxiliaryLoss"]


class AutoAuxiliaryLoss(torch.autograd.Function):
    """Identity on ``activation`` that feeds a gradient of one into ``aux_loss`` during backward."""

    @staticmethod
    def forward(ctx, activation, aux_loss):  # type: ignore[override]
        ctx.save_for_backward(aux_loss)
        return activation

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        (aux_loss,) = ctx.saved_tensors
        return grad_output, torch.ones_like(aux_loss)


def attach_auxiliary_loss(activation: torch.Tensor, aux_loss: torch.Tensor) -> torch.Tensor:
    """
    Tie ``aux_loss`` to ``activation`` so that ``backward`` through the activation also back-propagates the
    auxiliary loss (src/olmo_core/ops/__init__.py:4-28). Returns the activation unchanged.
    """
    return AutoAuxiliaryLoss.apply(activation, aux_loss)
