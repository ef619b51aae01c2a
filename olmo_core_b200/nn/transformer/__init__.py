"""Transformer models, blocks and configs (src/olmo_core/nn/transformer/__init__.py:25)."""

from .block import (
    LayerNormScaledTransformerBlock, MoEHybridReorderedNormTransformerBlock, MoEHybridTransformerBlock,
    MoEHybridTransformerBlockBase, MoEReorderedNormTransformerBlock, MoETransformerBlock,
    NormalizedTransformerBlock, PeriNormTransformerBlock, ReorderedNormTransformerBlock, TransformerBlock,
    TransformerBlockBase,
)
from .config import (
    TransformerActivationCheckpointingMode, TransformerBlockConfig, TransformerBlockType, TransformerConfig,
    TransformerDataParallelWrappingStrategy, TransformerType,
)
from .init import InitMethod
from .model import MoETransformer, NormalizedTransformer, Transformer

__all__ = [
    "InitMethod", "LayerNormScaledTransformerBlock", "MoEHybridReorderedNormTransformerBlock",
    "MoEHybridTransformerBlock", "MoEHybridTransformerBlockBase", "MoEReorderedNormTransformerBlock",
    "MoETransformer", "MoETransformerBlock", "NormalizedTransformer", "NormalizedTransformerBlock",
    "PeriNormTransformerBlock", "ReorderedNormTransformerBlock", "Transformer",
    "TransformerActivationCheckpointingMode", "TransformerBlock", "TransformerBlockBase",
    "TransformerBlockConfig", "TransformerBlockType", "TransformerConfig",
    "TransformerDataParallelWrappingStrategy", "TransformerType",
]
