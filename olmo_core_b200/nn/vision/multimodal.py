"""
Vision-language model: vision encoder + connector + language model
(role of src/olmo_core/nn/vision/multimodal.py:20-205). Projected image features are ADDED to the token embeddings at
the positions of the ``<im_patch>`` placeholder token; the data pipeline inserts exactly one placeholder per pooled feature.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ...config import Config
from ..transformer import TransformerConfig
from .config import VisionEncoderConfig
from .connector import VisionConnectorConfig

__all__ = ["MultimodalLMConfig", "MultimodalLM"]


@dataclass
class MultimodalLMConfig(Config):
    lm: TransformerConfig
    vision: VisionEncoderConfig
    connector: VisionConnectorConfig
    image_patch_token_id: int = 0
    vit_layers: Tuple[int, ...] = (-1,)  # hidden states to concatenate; needs connector.num_input_layers == len(vit_layers)

    def build(self, init_device: str = "cpu") -> "MultimodalLM":
        return MultimodalLM(self, init_device=init_device)


class MultimodalLM(nn.Module):
    def __init__(self, cfg: MultimodalLMConfig, init_device: str = "cpu"):
        super().__init__()
        if len(cfg.vit_layers) != cfg.connector.num_input_layers:
            raise ValueError("connector.num_input_layers must equal the number of selected ViT layers")
        self.cfg = cfg
        self.lm = cfg.lm.build(init_device=init_device)
        self.vision = cfg.vision.build(init_device=init_device)
        self.connector = cfg.connector.build(init_device=init_device)

    def _encode_images(self, images: torch.Tensor, pooled_patches_idx: torch.Tensor) -> torch.Tensor:
        """``images [B, crops, patches, patch_dim]`` → pooled features ``[B, n_pooled, d_model]``."""
        B, crops, patches, _ = images.shape
        states = self.vision(images.reshape(B * crops, patches, -1))
        picked = [states[i] for i in self.cfg.vit_layers]
        feats = picked[0] if len(picked) == 1 else torch.cat(picked, dim=-1)
        feats = feats[:, getattr(self.vision, "num_prefix_tokens", 0):]
        return self.connector(feats.reshape(B, crops * feats.shape[1], feats.shape[-1]), pooled_patches_idx)

    def forward(self, input_ids: torch.Tensor, images: Optional[torch.Tensor] = None,
                pooled_patches_idx: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None, **kwargs):
        if self.lm.embeddings is None:
            raise RuntimeError("MultimodalLM requires the LM to have an embedding table")
        device = self.lm.device
        input_ids = input_ids.to(device)
        labels = None if labels is None else labels.to(device)
        h = self.lm.embeddings(input_ids)
        if self.lm.embed_scale is not None:
            h = h * self.lm.embed_scale
        if self.lm.embedding_norm is not None:
            h = self.lm.embedding_norm(h)
        if images is not None:
            if pooled_patches_idx is None:
                raise ValueError("`pooled_patches_idx` is required when `images` is provided")
            feats = self._encode_images(images.to(device), pooled_patches_idx.to(device))
            at = (input_ids == self.cfg.image_patch_token_id).reshape(-1)
            n_slots, n_feats = int(at.sum()), feats.shape[0] * feats.shape[1]
            if n_slots != n_feats:
                raise ValueError(f"Number of <im_patch> tokens in input_ids ({n_slots}) does not match the number of "
                                 f"projected image features ({n_feats}).")
            d = h.shape[-1]
            flat = h.reshape(-1, d)
            h = flat.index_add(0, at.nonzero(as_tuple=True)[0], feats.reshape(-1, d).to(flat.dtype)).view(h.shape)
        return self.lm(input_ids, input_embeddings=h, labels=labels, **kwargs)
