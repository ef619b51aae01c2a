"""Residual addition as a module so that hooks can observe it (src/olmo_core/nn/residual_stream.py:5-19)."""

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["ResidualStream"]


class ResidualStream(nn.Module):
    def __init__(self, *, alpha: float = 1.0, dropout: float = 0.0):
        super().__init__()
        self.alpha = alpha
        self.dropout = dropout

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self.dropout > 0.0:
            y = F.dropout(y, p=self.dropout, training=self.training)
        return x + y if self.alpha == 1.0 else x + self.alpha * y
