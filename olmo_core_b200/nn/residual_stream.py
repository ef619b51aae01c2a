"""Residual addition as a module so that hooks can observe it (src/olmo_core/nn/residual_stream.py:5-19)."""

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["ResidualStream"]


class ResidualStream(nn.Module):
    def __init__(self, alpha: float = 1.0, dropout: float = 0.0):
        super().__init__()
        self.alpha = alpha
        self.dropout = dropout

    def forward(self, residual: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """``residual + alpha * dropout(x)``"""
        if self.dropout > 0.0:
            x = F.dropout(x, p=self.dropout, training=self.training)
        return residual + x if self.alpha == 1.0 else torch.add(residual, x, alpha=self.alpha)
