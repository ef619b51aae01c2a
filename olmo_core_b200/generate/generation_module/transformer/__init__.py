from .config import TransformerGenerationModuleConfig
from .generation_module import TransformerGenerationModule

__all__ = ["TransformerGenerationModule", "TransformerGenerationModuleConfig"]
