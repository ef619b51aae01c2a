from .config import GenerationConfig
from .generation_module import GenerationModule
from .transformer.config import TransformerGenerationModuleConfig
from .transformer.generation_module import TransformerGenerationModule

__all__ = ["GenerationConfig", "GenerationModule", "TransformerGenerationModule", "TransformerGenerationModuleConfig"]
