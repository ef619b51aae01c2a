"""Functional forms of the loss and normalisation ops (src/olmo_core/nn/functional/__init__.py:9)."""

from .cross_entropy_loss import cross_entropy_loss, fused_linear_cross_entropy_loss
from ..layer_norm import l2_normalize

__all__ = ["cross_entropy_loss", "fused_linear_cross_entropy_loss", "l2_normalize"]
