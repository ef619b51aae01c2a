"""Vision encoder, connector and multimodal wrapper for vision-language training (src/olmo_core/nn/vision/__init__.py)."""

from .config import VisionBlockConfig, VisionBlockType, VisionEncoderConfig, VisionEncoderType
from .connector import ImagePoolingType, ImageProjectorType, VisionConnector, VisionConnectorConfig
from .image_vit import VisionTransformer, ViTAttention, ViTBlock, ViTMLP
from .multimodal import MultimodalLM, MultimodalLMConfig

__all__ = ["VisionEncoderType", "VisionEncoderConfig", "VisionBlockType", "VisionBlockConfig", "ViTAttention", "ViTMLP",
           "ViTBlock", "VisionTransformer", "ImagePoolingType", "ImageProjectorType", "VisionConnectorConfig",
           "VisionConnector", "MultimodalLMConfig", "MultimodalLM"]
