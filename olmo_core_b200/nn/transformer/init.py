"""
Weight-initialisation schemes (behaviour of src/olmo_core/nn/transformer/init.py:16-254).

Every scheme is a table from a parameter's *role* to the standard deviation of a normal distribution
truncated at three sigma. Draws are made from one seeded generator in a fixed module order, and a
sharded parameter always draws the full tensor and keeps its slice, so the resulting model does not
depend on how it is sharded.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Optional

import torch
import torch.nn as nn

from ...config import StrEnum
from ...distributed.utils import distribute_like, get_local_tensor

try:
    from torch.distributed.tensor import DTensor
except ImportError:  # pragma: no cover
    DTensor = None  # type: ignore

if TYPE_CHECKING:
    from ..feed_forward import FeedForward

__all__ = ["InitMethod", "init_linear", "init_tensor_"]


def init_tensor_(x: torch.Tensor, *, std: Optional[float], generator: Optional[torch.Generator] = None,
                 truncate: bool = True, mean: float = 0.0) -> None:
    """Fill ``x`` from N(mean, std) (truncated at 3 sigma unless ``truncate`` is False), shard-invariantly."""
    std = 1.0 if std is None else std

    def fill(t: torch.Tensor) -> None:
        if truncate:
            nn.init.trunc_normal_(t, mean=mean, std=std, a=mean - 3 * std, b=mean + 3 * std, generator=generator)
        else:
            nn.init.normal_(t, mean=mean, std=std, generator=generator)

    with torch.no_grad():
        if DTensor is not None and isinstance(x, DTensor):
            full = torch.zeros(x.shape, dtype=x.dtype, device=x.device)
            fill(full)
            get_local_tensor(x).copy_(get_local_tensor(distribute_like(x, full)))
            return
        shard_info = getattr(x, "_shard_info", None)
        if shard_info is not None:
            # Parameter owned by the sharded-parameter runtime: draw the full tensor, keep our rows.
            full = torch.zeros(shard_info.full_shape, dtype=x.dtype, device=x.device)
            fill(full)
            real = max(0, min(x.shape[0], shard_info.full_shape[0] - shard_info.row_start))  # the rest is padding
            if real > 0:
                x[:real].copy_(full.narrow(0, shard_info.row_start, real))
            if real < x.shape[0]:
                x[real:].zero_()
            return
        fill(x)


def init_linear(m: nn.Module, *, std: float = 0.02, generator: Optional[torch.Generator] = None) -> None:
    init_tensor_(m.weight, std=std, generator=generator)
    if getattr(m, "bias", None) is not None:
        with torch.no_grad():
            m.bias.zero_()


class InitMethod(StrEnum):
    normal = "normal"
    """Every matrix from N(0, std) truncated at 3 sigma."""
    normalized = "normalized"
    """nGPT: std = d_model^-1/2, output projections additionally divided by sqrt(2 * n_layers)."""
    llama = "llama"
    """Embeddings N(0,1); attention output and the MLP's w3/w2 divided by sqrt(2 * n_layers); head d_model^-1/2."""
    llama_depth = "llama_depth"
    """As ``llama`` with the divisor sqrt(2 * (layer index + 1))."""
    fan_in = "fan_in"
    """std = fan_in^-1/2 per matrix; embeddings N(0, 1/embed_scale)."""

    # -- helpers ------------------------------------------------------------------------------------
    def _depth_divisor(self, block_idx: int, num_blocks: int) -> float:
        if self == InitMethod.llama_depth:
            return (2 * (block_idx + 1)) ** 0.5
        return (2 * num_blocks) ** 0.5

    def init_embeddings(self, m: nn.Module, *, d_model: int, embed_scale: Optional[float] = None, std: float = 0.02,
                        generator: Optional[torch.Generator] = None) -> None:
        if self in (InitMethod.llama, InitMethod.llama_depth):
            init_tensor_(m.weight, std=1.0, generator=generator, truncate=False)
        elif self == InitMethod.normalized:
            init_tensor_(m.weight, std=d_model**-0.5, generator=generator, truncate=False)
        elif self == InitMethod.fan_in:
            init_tensor_(m.weight, std=1.0 / embed_scale if embed_scale is not None else 1.0, generator=generator,
                         truncate=False)
        else:
            init_tensor_(m.weight, std=std, generator=generator)

    def init_final_w_out(self, m: nn.Module, *, d_model: int, std: float = 0.02,
                         generator: Optional[torch.Generator] = None) -> None:
        if self != InitMethod.normal:
            std = d_model**-0.5
        init_linear(m, std=std, generator=generator)

    def attention_stds(self, *, d_model: int, in_features: int, out_in_features: int, block_idx: int, num_blocks: int,
                       std: float):
        """(std of the q/k/v/gate projections, std of the output projection)."""
        if self == InitMethod.fan_in:
            return in_features**-0.5, out_in_features**-0.5
        if self == InitMethod.normalized:
            base = d_model**-0.5
            return base, base / (2 * num_blocks) ** 0.5
        if self in (InitMethod.llama, InitMethod.llama_depth):
            return std, std / self._depth_divisor(block_idx, num_blocks)
        return std, std

    def init_attention(self, m: nn.Module, *, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                       generator: Optional[torch.Generator] = None) -> None:
        m.init_weights(init_method=self, d_model=d_model, block_idx=block_idx, num_blocks=num_blocks, std=std,
                       generator=generator)

    def init_feed_forward(self, m: "FeedForward", *, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                          generator: Optional[torch.Generator] = None) -> None:
        if self == InitMethod.fan_in:
            s1, s3, s2 = m.w1.in_features**-0.5, m.w3.in_features**-0.5, m.w2.in_features**-0.5
        elif self == InitMethod.normalized:
            s1 = s3 = d_model**-0.5
            s2 = s3 / (2 * num_blocks) ** 0.5
        elif self in (InitMethod.llama, InitMethod.llama_depth):
            s1 = std
            s3 = s2 = std / self._depth_divisor(block_idx, num_blocks)
        else:
            s1 = s3 = s2 = std
        init_linear(m.w1, std=s1, generator=generator)
        init_linear(m.w3, std=s3, generator=generator)
        init_linear(m.w2, std=s2, generator=generator)

    def init_feed_forward_moe(self, m: nn.Module, *, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                              generator: Optional[torch.Generator] = None) -> None:
        mlp = m.experts.mlp
        if self in (InitMethod.llama, InitMethod.llama_depth):
            std = std / self._depth_divisor(block_idx, num_blocks)
        if self == InitMethod.fan_in:
            s_router, s1, s2, s3 = d_model**-0.5, mlp.d_model**-0.5, mlp.hidden_size**-0.5, mlp.d_model**-0.5
        else:
            s_router = s1 = s2 = s3 = std
        init_tensor_(m.router.weight, std=s_router, generator=generator)
        init_tensor_(mlp.w1, std=s1, generator=generator)
        init_tensor_(mlp.w2, std=s2, generator=generator)
        init_tensor_(mlp.w3, std=s3, generator=generator)
        shared = getattr(m, "shared_mlp", None)
        if shared is not None:
            self.init_feed_forward(shared, d_model=d_model, block_idx=block_idx, num_blocks=num_blocks, std=std,
                                   generator=generator)
