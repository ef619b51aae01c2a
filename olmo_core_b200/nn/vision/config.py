"""
Vision-encoder configuration (names and presets of src/olmo_core/nn/vision/config.py:18-416). One ViT implementation
covers the CLIP family (class token, pre-LayerNorm, no patch-embedding bias) and the SigLIP / SigLIP2 families (patches
only); the named presets differ in sizes only and are generated from one table.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple

import torch.nn as nn

from ...config import DType, StrEnum
from ..config import ModuleConfig

__all__ = ["VisionEncoderType", "VisionBlockType", "VisionBlockConfig", "VisionEncoderConfig"]


class VisionEncoderType(StrEnum):
    openai = "openai"  # CLIP ViT (class token); the defaults are ViT-L/14-336
    siglip = "siglip"  # no class token
    siglip2 = "siglip2"  # same architecture as SigLIP


class VisionBlockType(StrEnum):
    standard = "standard"  # pre-LN block: attention + MLP, each with a residual


@dataclass
class VisionBlockConfig(ModuleConfig):
    name: VisionBlockType = VisionBlockType.standard

    def build(self, cfg: "VisionEncoderConfig", init_device: str = "cpu") -> nn.Module:
        from .image_vit import ViTBlock

        if self.name == VisionBlockType.standard:
            return ViTBlock(cfg, init_device=init_device)
        raise NotImplementedError(self.name)


# name -> (family, input size, patch, width, heads, layers, head_dim, mlp width); positions = (input / patch)^2
_SIGLIP_PRESETS = {
    "siglip_b16_224": ("siglip", 224, 16, 768, 12, 12, 64, 3072),
    "siglip_l16_384": ("siglip", 384, 16, 1024, 16, 24, 64, 4096),
    "siglip_so400m_patch14_224": ("siglip", 224, 14, 1152, 16, 27, 72, 4304),
    "siglip_so400m": ("siglip", 378, 14, 1152, 16, 27, 72, 4304),
    "siglip2_b16_256": ("siglip2", 256, 16, 768, 12, 12, 64, 3072),
    "siglip2_l16_256": ("siglip2", 256, 16, 1024, 16, 24, 64, 4096),
    "siglip2_so400m_patch14_378": ("siglip2", 378, 14, 1152, 16, 27, 72, 4304),
    "siglip2_so400m_patch16_256": ("siglip2", 256, 16, 1152, 16, 27, 72, 4304),
}


@dataclass
class VisionEncoderConfig(ModuleConfig):
    name: VisionEncoderType = VisionEncoderType.openai
    image_default_input_size: Tuple[int, int] = (336, 336)
    image_patch_size: int = 14
    image_emb_dim: int = 1024
    image_num_heads: int = 16
    image_num_key_value_heads: int = 16
    image_num_layers: int = 23  # the last CLIP layer is never used downstream, so it is not built
    image_head_dim: int = 64
    image_mlp_dim: int = 4096
    image_mlp_activations: str = "quick_gelu"
    image_num_pos: int = 577  # 24 x 24 patches + class token
    image_norm_eps: float = 1e-5
    attention_dropout: float = 0.0
    residual_dropout: float = 0.0
    use_cls_token: bool = True
    patch_embedding_bias: bool = False
    use_pre_ln: bool = True
    block: VisionBlockConfig = field(default_factory=VisionBlockConfig)
    initializer_range: float = 0.02
    dtype: DType = DType.float32

    @property
    def image_num_patch(self) -> Tuple[int, int]:
        h, w = self.image_default_input_size
        return h // self.image_patch_size, w // self.image_patch_size

    @classmethod
    def _siglip(cls, key: str) -> "VisionEncoderConfig":
        family, size, patch, width, heads, layers, head_dim, mlp = _SIGLIP_PRESETS[key]
        return cls(name=VisionEncoderType(family), use_cls_token=False, patch_embedding_bias=True, use_pre_ln=False,
                   image_default_input_size=(size, size), image_patch_size=patch, image_emb_dim=width,
                   image_num_heads=heads, image_num_key_value_heads=heads, image_num_layers=layers,
                   image_head_dim=head_dim, image_mlp_dim=mlp, image_mlp_activations="gelu_pytorch_tanh",
                   image_num_pos=(size // patch) ** 2, image_norm_eps=1e-6)

    def build(self, init_device: str = "cpu") -> nn.Module:
        from .image_vit import VisionTransformer

        return VisionTransformer(self, init_device=init_device)


def _preset(key: str):
    def factory(cls) -> VisionEncoderConfig:
        return cls._siglip(key)

    factory.__name__ = key
    factory.__doc__ = f"Sizes of the '{key}' checkpoint family."
    return classmethod(factory)


for _key in _SIGLIP_PRESETS:
    setattr(VisionEncoderConfig, _key, _preset(_key))
