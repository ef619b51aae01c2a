"""Format-independent machinery for converting named state (API of src/olmo_core/nn/conversion/__init__.py)."""

from .state_converter import StateConverter
from .state_mapping import StateMapping, StateMappingTemplate, StateType, TemplatePlaceholder

__all__ = ["StateConverter", "StateMapping", "StateMappingTemplate", "StateType", "TemplatePlaceholder"]
