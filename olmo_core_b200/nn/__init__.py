"""Model building blocks: attention, RoPE, norms, MLPs, MoE, LM head, transformer models."""

_VISION_NAMES = ("VisionEncoderType", "VisionEncoderConfig", "VisionTransformer", "ImagePoolingType", "ImageProjectorType",
                 "VisionConnectorConfig", "VisionConnector", "MultimodalLMConfig", "MultimodalLM")

__all__ = list(_VISION_NAMES)


def __getattr__(name: str):
    # the vision classes are re-exported here as in src/olmo_core/nn/__init__.py, resolved on first use
    if name in _VISION_NAMES:
        from . import vision

        return getattr(vision, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
