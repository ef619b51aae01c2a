"""Depth-wise causal 1-D convolution ("short convolution") used by linear-attention mixers (src/olmo_core/nn/convolution.py)."""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["CausalConv1d"]


class CausalConv1d(nn.Conv1d):
    """
    ``y[t, c] = act(sum_j w[c, j] * x[t - (K-1) + j, c] + b[c])`` over ``[B, T, C]`` inputs. With ``cu_seqlens`` (batch
    size 1, packed documents) the window never reaches across a document boundary.
    """

    def __init__(self, *, hidden_size: int, kernel_size: int, bias: bool = False, backend: str = "cuda",
                 dtype: Optional[torch.dtype] = None, init_device: str = "cpu", activation: Optional[str] = "silu"):
        super().__init__(in_channels=hidden_size, out_channels=hidden_size, kernel_size=kernel_size, groups=hidden_size,
                         bias=bias, padding=kernel_size - 1, device=init_device, dtype=dtype)
        self.hidden_size = hidden_size
        self.backend = backend
        self.activation = activation
        self.cp_enabled = False
        self._cp_channel_slice: Optional[slice] = None

    def forward(self, x: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:  # type: ignore[override]
        weight, bias = self.weight, self.bias
        if self.cp_enabled and self._cp_channel_slice is not None:
            weight = weight[self._cp_channel_slice]
            bias = None if bias is None else bias[self._cp_channel_slice]
        K = weight.shape[-1]
        T = x.shape[1]
        xt = x.transpose(1, 2)  # [B, C, T]
        if cu_seqlens is None:
            y = F.conv1d(xt, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), padding=K - 1,
                         groups=weight.shape[0])[..., :T]
        else:
            if x.shape[0] != 1:
                raise ValueError("'cu_seqlens' needs batch size 1")
            bounds = cu_seqlens.tolist()
            parts = [F.conv1d(xt[..., a:b], weight.to(x.dtype), None if bias is None else bias.to(x.dtype), padding=K - 1,
                              groups=weight.shape[0])[..., : b - a] for a, b in zip(bounds[:-1], bounds[1:])]
            y = torch.cat(parts, dim=-1)
        y = y.transpose(1, 2)
        if self.activation in ("silu", "swish"):
            y = F.silu(y)
        return y

    def apply_cp(self, cp_mesh) -> None:
        """Ulysses-style channel parallelism: keep all parameters, use this rank's slice of the channels in forward."""
        if cp_mesh.size() == 1:
            return
        n = self.hidden_size // cp_mesh.size()
        start = cp_mesh.get_local_rank() * n
        self._cp_channel_slice = slice(start, start + n)
        self.cp_enabled = True
