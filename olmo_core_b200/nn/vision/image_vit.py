"""
Vision transformer over pre-patchified images (role of src/olmo_core/nn/vision/image_vit.py:18-311). ``forward`` returns
the hidden state after EVERY block so that callers can pick layers (e.g. ``[-2, -9]``). Attention is bidirectional and
runs through this package's attention op; the projections are the same ``Linear`` modules the language model uses.
"""

from __future__ import annotations

import math
from typing import Callable, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.attention import attention
from ..feed_forward import Linear
from .config import VisionEncoderConfig

__all__ = ["ViTAttention", "ViTMLP", "ViTBlock", "VisionTransformer"]


def _activation(name: str) -> Callable[[torch.Tensor], torch.Tensor]:
    table = {
        "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x),
        "gelu": F.gelu,
        "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh"),
        "silu": F.silu,
    }
    if name not in table:
        raise ValueError(f"unknown activation '{name}'")
    return table[name]


def _normal_(linear: nn.Module, std: float) -> None:
    nn.init.normal_(linear.weight, std=std)
    if linear.bias is not None:
        nn.init.zeros_(linear.bias)


class ViTAttention(nn.Module):
    def __init__(self, cfg: VisionEncoderConfig, init_device: str = "cpu"):
        super().__init__()
        dtype = cfg.dtype.as_pt()
        self.n_heads, self.n_kv_heads, self.head_dim = cfg.image_num_heads, cfg.image_num_key_value_heads, cfg.image_head_dim
        self.std = cfg.initializer_range
        d = cfg.image_emb_dim
        self.wq = Linear(d, self.n_heads * self.head_dim, True, dtype, init_device)
        self.wk = Linear(d, self.n_kv_heads * self.head_dim, True, dtype, init_device)
        self.wv = Linear(d, self.n_kv_heads * self.head_dim, True, dtype, init_device)
        self.wo = Linear(self.n_heads * self.head_dim, d, True, dtype, init_device)
        self.attention_dropout = cfg.attention_dropout
        self.residual_dropout = nn.Dropout(cfg.residual_dropout)

    def reset_parameters(self) -> None:
        for w in (self.wq, self.wk, self.wv, self.wo):
            _normal_(w, self.std)

    def forward(self, x: torch.Tensor, kv: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Self-attention over ``x [B, N, D]``, or cross-attention onto ``kv [B, M, D]``."""
        src = x if kv is None else kv
        B, N, _ = x.shape
        q = self.wq(x).view(B, N, self.n_heads, self.head_dim)
        k = self.wk(src).view(B, src.shape[1], self.n_kv_heads, self.head_dim)
        v = self.wv(src).view(B, src.shape[1], self.n_kv_heads, self.head_dim)
        out = attention(q, k, v, causal=False, dropout_p=self.attention_dropout if self.training else 0.0)
        return self.residual_dropout(self.wo(out.reshape(B, N, -1)))


class ViTMLP(nn.Module):
    def __init__(self, cfg: VisionEncoderConfig, init_device: str = "cpu"):
        super().__init__()
        dtype = cfg.dtype.as_pt()
        self.w1 = Linear(cfg.image_emb_dim, cfg.image_mlp_dim, True, dtype, init_device)
        self.w2 = Linear(cfg.image_mlp_dim, cfg.image_emb_dim, True, dtype, init_device)
        self.act = _activation(cfg.image_mlp_activations)
        self.std = cfg.initializer_range

    def reset_parameters(self) -> None:
        _normal_(self.w1, self.std)
        _normal_(self.w2, self.std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w2(self.act(self.w1(x)))


class ViTBlock(nn.Module):
    def __init__(self, cfg: VisionEncoderConfig, init_device: str = "cpu"):
        super().__init__()
        dtype = cfg.dtype.as_pt()
        self.attention = ViTAttention(cfg, init_device)
        self.feed_forward = ViTMLP(cfg, init_device)
        self.attention_norm = nn.LayerNorm(cfg.image_emb_dim, eps=cfg.image_norm_eps, device=init_device, dtype=dtype)
        self.ffn_norm = nn.LayerNorm(cfg.image_emb_dim, eps=cfg.image_norm_eps, device=init_device, dtype=dtype)

    def reset_parameters(self) -> None:
        self.attention.reset_parameters()
        self.feed_forward.reset_parameters()
        self.attention_norm.reset_parameters()
        self.ffn_norm.reset_parameters()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attention(self.attention_norm(x))
        return x + self.feed_forward(self.ffn_norm(x))


def _interpolate_pos_emb(pos_emb: torch.Tensor, patch_num: Tuple[int, int], num_prefix: int) -> torch.Tensor:
    """Resize the (square) grid of learned positions to ``patch_num`` with bicubic interpolation; prefix rows are kept."""
    prefix, grid = pos_emb[:num_prefix], pos_emb[num_prefix:]
    side = int(math.isqrt(grid.shape[0]))
    if side * side != grid.shape[0]:
        raise ValueError("the positional embedding does not describe a square grid")
    if (side, side) != tuple(patch_num):
        g = grid.view(1, side, side, -1).permute(0, 3, 1, 2).float()
        g = F.interpolate(g, size=tuple(patch_num), mode="bicubic", align_corners=False, antialias=True)
        grid = g.permute(0, 2, 3, 1).reshape(-1, pos_emb.shape[-1]).to(pos_emb.dtype)
    return torch.cat([prefix, grid], dim=0) if num_prefix else grid


class VisionTransformer(nn.Module):
    def __init__(self, cfg: VisionEncoderConfig, init_device: str = "cpu"):
        super().__init__()
        self.cfg = cfg
        dtype = cfg.dtype.as_pt()
        self.num_prefix_tokens = 1 if cfg.use_cls_token else 0
        self.patch_embedding = Linear(cfg.image_patch_size ** 2 * 3, cfg.image_emb_dim, cfg.patch_embedding_bias, dtype,
                                      init_device)
        self.class_embedding = (nn.Parameter(torch.zeros(cfg.image_emb_dim, device=init_device, dtype=dtype))
                                if cfg.use_cls_token else None)
        self.positional_embedding = nn.Parameter(torch.zeros(cfg.image_num_pos, cfg.image_emb_dim, device=init_device,
                                                             dtype=dtype))
        self.pre_ln = (nn.LayerNorm(cfg.image_emb_dim, eps=cfg.image_norm_eps, device=init_device, dtype=dtype)
                       if cfg.use_pre_ln else None)
        self.blocks = nn.ModuleList([cfg.block.build(cfg, init_device=init_device) for _ in range(cfg.image_num_layers)])
        if init_device != "meta":
            self.reset_parameters()

    def reset_parameters(self) -> None:
        scale = self.cfg.image_emb_dim ** -0.5
        if self.class_embedding is not None:
            nn.init.normal_(self.class_embedding, std=scale)
        nn.init.normal_(self.positional_embedding, std=scale)
        _normal_(self.patch_embedding, 0.02)
        if self.pre_ln is not None:
            self.pre_ln.reset_parameters()
        for block in self.blocks:
            block.reset_parameters()

    def forward(self, x: torch.Tensor, patch_num: Optional[Tuple[int, int]] = None) -> List[torch.Tensor]:
        """``x [B, n_patches, patch_size^2 * 3]`` → one ``[B, prefix + n_patches, D]`` tensor per block."""
        patch_num = patch_num or self.cfg.image_num_patch
        h = self.patch_embedding(x)
        if self.class_embedding is not None:
            h = torch.cat([self.class_embedding.to(h.dtype).expand(h.shape[0], 1, -1), h], dim=1)
        h = h + _interpolate_pos_emb(self.positional_embedding, patch_num, self.num_prefix_tokens)[None].to(h.dtype)
        if self.pre_ln is not None:
            h = self.pre_ln(h)
        states: List[torch.Tensor] = []
        for block in self.blocks:
            h = block(h)
            states.append(h)
        return states
