"""Transformer models, blocks and configs (src/olmo_core/nn/transformer/__init__.py:25)."""

from .block import (
    LayerNormScaledTransformerBlock,
    MoEHybridReorderedNormTransformerBlock,
    MoEHybridTransformerBlock,
    MoEHybridTransformerBlockBase,
    MoEReorderedNormTransformerBlock,
    MoETransformerBlock,
    NormalizedTransformerBlock,
    PeriNormTransformerBlock,
    ReorderedNormTransformerBlock,
    TransformerBlock,
    TransformerBlockBase,
)
from .config import (
    TransformerActivationCheckpointingMode,
    TransformerBlockConfig,
    TransformerBlockType,
    TransformerConfig,
    TransformerDataParallelWrappingStrategy,
    TransformerType,
)
from .init import InitMethod
from .model import MoETransformer, NormalizedTransformer, Transformer

__all__ = [
    "TransformerType",
    "TransformerConfig",
    "Transformer",
    "NormalizedTransformer",
    "MoETransformer",
    "MoEHybridTransformerBlockBase",
    "MoEHybridTransformerBlock",
    "MoEHybridReorderedNormTransformerBlock",
    "TransformerBlockType",
    "TransformerBlockConfig",
    "TransformerBlockBase",
    "TransformerBlock",
    "ReorderedNormTransformerBlock",
    "LayerNormScaledTransformerBlock",
    "PeriNormTransformerBlock",
    "NormalizedTransformerBlock",
    "MoETransformerBlock",
    "MoEReorderedNormTransformerBlock",
    "TransformerDataParallelWrappingStrategy",
    "TransformerActivationCheckpointingMode",
    "InitMethod",
]
