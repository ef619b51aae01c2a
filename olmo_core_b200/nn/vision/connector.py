"""
Vision-to-language connector (role of src/olmo_core/nn/vision/connector.py:20-407): gathers the patch features of each
pool group (``pooled_patches_idx [B, n_pooled, pool_size]``, ``-1`` = padding), pools a group into one token by
cross-attention with the group mean as the query, and projects into the language model's width.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import DType, StrEnum
from ..config import ModuleConfig
from ..feed_forward import Linear
from .config import VisionEncoderConfig

__all__ = ["ImagePoolingType", "ImageProjectorType", "VisionConnectorConfig", "VisionConnector"]


class ImagePoolingType(StrEnum):
    attention_meanq = "attention_meanq"  # query = mean of the group, keys / values = the group's patches
    none = "none"  # pool_size must be 1


class ImageProjectorType(StrEnum):
    mlp = "mlp"  # SwiGLU: w2(silu(w1 x) * w3 x)
    linear = "linear"  # one bias-free projection


class _PoolingCrossAttention(nn.Module):
    def __init__(self, *, input_dim: int, emb_dim: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 initializer_range: float, dtype: torch.dtype, init_device: str):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.std = initializer_range
        self.wq = Linear(input_dim, num_heads * head_dim, True, dtype, init_device)
        self.wk = Linear(input_dim, num_kv_heads * head_dim, True, dtype, init_device)
        self.wv = Linear(input_dim, num_kv_heads * head_dim, True, dtype, init_device)
        self.wo = Linear(num_heads * head_dim, emb_dim, True, dtype, init_device)

    def reset_parameters(self) -> None:
        for w in (self.wq, self.wk, self.wv, self.wo):
            nn.init.normal_(w.weight, std=self.std)
            nn.init.zeros_(w.bias)

    def forward(self, query: torch.Tensor, context: torch.Tensor, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``query [G, 1, D_in]``, ``context [G, P, D_in]``, ``attn_mask [G, 1, 1, P]`` (True = attend) → ``[G, 1, D]``."""
        G, P = context.shape[0], context.shape[1]
        q = self.wq(query).view(G, 1, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.wk(context).view(G, P, self.num_kv_heads, self.head_dim).transpose(1, 2)
        v = self.wv(context).view(G, P, self.num_kv_heads, self.head_dim).transpose(1, 2)
        if self.num_kv_heads != self.num_heads:
            rep = self.num_heads // self.num_kv_heads
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask)
        return self.wo(out.transpose(1, 2).reshape(G, 1, -1))


class _ConnectorMLP(nn.Module):
    def __init__(self, input_dim: int, hidden: int, output_dim: int, std: float, dtype: torch.dtype, init_device: str):
        super().__init__()
        self.w1 = Linear(input_dim, hidden, False, dtype, init_device)
        self.w3 = Linear(input_dim, hidden, False, dtype, init_device)
        self.w2 = Linear(hidden, output_dim, False, dtype, init_device)
        self.std = std

    def reset_parameters(self) -> None:
        for w in (self.w1, self.w2, self.w3):
            nn.init.normal_(w.weight, std=self.std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


@dataclass
class VisionConnectorConfig(ModuleConfig):
    image_emb_dim: int = 1024
    image_num_heads: int = 16
    image_num_key_value_heads: int = 16
    image_head_dim: int = 64
    output_dim: int = 4096
    num_input_layers: int = 1  # ViT layers concatenated along the feature dimension in front of the pooling
    pooling_type: ImagePoolingType = ImagePoolingType.attention_meanq
    pooling_attention_mask: bool = False  # keep padded slots (-1) out of the pooling attention and of the mean query
    projector_type: ImageProjectorType = ImageProjectorType.mlp
    mlp_hidden_size: Optional[int] = None  # default 4 * image_emb_dim
    initializer_range: float = 0.02
    dtype: DType = DType.float32

    @classmethod
    def from_vision_encoder(cls, vision_cfg: VisionEncoderConfig, output_dim: int, num_input_layers: int = 1,
                            **kwargs) -> "VisionConnectorConfig":
        return cls(image_emb_dim=vision_cfg.image_emb_dim, image_num_heads=vision_cfg.image_num_heads,
                   image_num_key_value_heads=vision_cfg.image_num_key_value_heads,
                   image_head_dim=vision_cfg.image_head_dim, output_dim=output_dim, num_input_layers=num_input_layers,
                   dtype=vision_cfg.dtype, **kwargs)

    @property
    def pooling_input_dim(self) -> int:
        return self.num_input_layers * self.image_emb_dim

    @property
    def projector_input_dim(self) -> int:
        return self.pooling_input_dim if self.pooling_type == ImagePoolingType.none else self.image_emb_dim

    def build(self, init_device: str = "cpu") -> "VisionConnector":
        return VisionConnector(self, init_device=init_device)


class VisionConnector(nn.Module):
    def __init__(self, cfg: VisionConnectorConfig, init_device: str = "cpu"):
        super().__init__()
        self.cfg = cfg
        dtype = cfg.dtype.as_pt()
        self.pooling: Optional[_PoolingCrossAttention] = None
        if cfg.pooling_type == ImagePoolingType.attention_meanq:
            self.pooling = _PoolingCrossAttention(
                input_dim=cfg.pooling_input_dim, emb_dim=cfg.image_emb_dim, num_heads=cfg.image_num_heads,
                num_kv_heads=cfg.image_num_key_value_heads, head_dim=cfg.image_head_dim,
                initializer_range=cfg.initializer_range, dtype=dtype, init_device=init_device)
        if cfg.projector_type == ImageProjectorType.mlp:
            self.projector: nn.Module = _ConnectorMLP(cfg.projector_input_dim, cfg.mlp_hidden_size or 4 * cfg.image_emb_dim,
                                                      cfg.output_dim, cfg.initializer_range, dtype, init_device)
        elif cfg.projector_type == ImageProjectorType.linear:
            self.projector = Linear(cfg.projector_input_dim, cfg.output_dim, False, dtype, init_device)
        else:
            raise NotImplementedError(cfg.projector_type)
        if init_device != "meta":
            self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.pooling is not None:
            self.pooling.reset_parameters()
        if isinstance(self.projector, _ConnectorMLP):
            self.projector.reset_parameters()
        else:
            nn.init.normal_(self.projector.weight, std=self.cfg.initializer_range)

    def forward(self, image_features: torch.Tensor, pooled_patches_idx: torch.Tensor) -> torch.Tensor:
        """``image_features [B, n_patches_total, D_in]``, ``pooled_patches_idx [B, n_pooled, pool]`` → ``[B, n_pooled, out]``."""
        cfg = self.cfg
        B, _, dim = image_features.shape
        n_pooled, pool = pooled_patches_idx.shape[1:]
        valid = pooled_patches_idx >= 0
        rows = torch.arange(B, device=image_features.device).view(B, 1, 1).expand(B, n_pooled, pool)
        groups = image_features[rows, pooled_patches_idx.clamp(min=0)] * valid.unsqueeze(-1).to(image_features.dtype)
        if cfg.pooling_type == ImagePoolingType.none:
            if pool != 1:
                raise ValueError("pool_size must be 1 when pooling_type=none")
            pooled = groups.view(B, n_pooled, dim)
        else:
            assert self.pooling is not None
            flat = groups.view(B * n_pooled, pool, dim)
            mask = None
            if cfg.pooling_attention_mask:
                flat_valid = valid.view(B * n_pooled, pool)
                mask = flat_valid.view(B * n_pooled, 1, 1, pool)
                query = flat.sum(dim=1, keepdim=True) / flat_valid.sum(-1).clamp(min=1).view(-1, 1, 1).to(flat.dtype)
            else:
                query = flat.mean(dim=1, keepdim=True)
            pooled = self.pooling(query, flat, attn_mask=mask).view(B, n_pooled, cfg.image_emb_dim)
        return self.projector(pooled)
