"""Cross-entropy (+ z-loss) as a module (src/olmo_core/nn/cross_entropy_loss.py)."""

from __future__ import annotations

from typing import Literal, Optional, Tuple

import torch
import torch.nn as nn

from .functional import cross_entropy_loss

__all__ = ["CrossEntropyLoss"]


class CrossEntropyLoss(nn.Module):
    """
    ``forward(logits [..., V], labels [...]) -> (ce_loss, z_loss | None)`` with ``ignore_index`` masking, ``sum`` /
    ``mean`` / ``none`` reduction and ``z_loss_multiplier * logsumexp(logits)**2`` as the auxiliary z-loss.
    """

    def __init__(self, *, ignore_index: int = -100, reduction: Literal["mean", "sum", "none"] = "mean",
                 z_loss_multiplier: Optional[float] = None, compile: bool = False, fused: bool = False):
        super().__init__()
        del compile  # no tracing compiler here; 'fused' selects the row kernel, which is already the CUDA default
        self.ignore_index = ignore_index
        self._reduction = reduction
        self.z_loss_multiplier = z_loss_multiplier
        self.fused = fused
        self._tp_enabled = False

    @property
    def compile_enabled(self) -> bool:
        return False

    @property
    def tp_enabled(self) -> bool:
        return self._tp_enabled

    @property
    def z_loss_enabled(self) -> bool:
        return self.z_loss_multiplier is not None

    @property
    def reduction(self) -> str:
        return self._reduction

    def forward(self, logits: torch.Tensor, labels: torch.Tensor,
                div_factor: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        flat_logits = logits.reshape(-1, logits.shape[-1])
        flat_labels = labels.reshape(-1)
        reduction = "sum" if (self._reduction == "mean" and div_factor is not None) else self._reduction
        ce, z = cross_entropy_loss(flat_logits, flat_labels, ignore_index=self.ignore_index, reduction=reduction,
                                   compute_z_loss=self.z_loss_enabled, z_loss_multiplier=self.z_loss_multiplier or 1e-4)
        if div_factor is not None and self._reduction == "mean":
            ce = ce / div_factor
            z = None if z is None else z / div_factor
        if self._reduction == "none":
            ce = ce.view(labels.shape)
            z = None if z is None else z.view(labels.shape)
        return ce, z

    def apply_tp(self, tp_mesh, input_layouts=None, shard_dimension: int = 1, output_layout=None,
                 use_local_output: bool = False) -> None:
        """Logits reach this module gathered over the sequence (see ``parallel.tensor``); nothing to shard."""
        del tp_mesh, input_layouts, shard_dimension, output_layout, use_local_output
        self._tp_enabled = True
