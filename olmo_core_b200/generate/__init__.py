"""Text generation: sampling, KV-cached decoding and a chat CLI (``python -m olmo_core_b200.generate.chat``)."""

from .generation_module import (
    GenerationConfig,
    GenerationModule,
    TransformerGenerationModule,
    TransformerGenerationModuleConfig,
)

__all__ = ["GenerationConfig", "GenerationModule", "TransformerGenerationModule", "TransformerGenerationModuleConfig"]
