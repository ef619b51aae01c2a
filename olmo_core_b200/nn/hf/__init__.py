"""
Conversion between this framework's transformers and Hugging Face causal LMs (public names of
src/olmo_core/nn/hf/__init__.py). The name mapping is the table ``OLMO_CORE_TO_HF_TEMPLATES`` in
:mod:`olmo_core_b200.nn.hf.convert`.
"""

from .checkpoint import load_hf_model, save_hf_model
from .config import get_hf_config
from .convert import (
    convert_state_from_hf,
    convert_state_to_hf,
    get_converter_from_hf,
    get_converter_to_hf,
)
from .convert_checkpoint import convert_checkpoint_to_hf, load_config, validate_conversion

from .hybrid import (
    convert_hybrid_state_to_hf,
    convert_qwen3_5_state_from_hf,
    get_hybrid_hf_config,
    get_hybrid_layer_types,
    is_olmo_hybrid_model,
    save_hf_hybrid_model,
)

__all__ = ["convert_hybrid_state_to_hf", "convert_qwen3_5_state_from_hf", "get_hybrid_hf_config", "get_hybrid_layer_types",
           "is_olmo_hybrid_model", "save_hf_hybrid_model", "convert_checkpoint_to_hf", "convert_state_from_hf", "convert_state_to_hf", "get_converter_from_hf",
           "get_converter_to_hf", "get_hf_config", "load_config", "load_hf_model", "save_hf_model", "validate_conversion"]
