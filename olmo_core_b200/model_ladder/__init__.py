"""
Model ladders: a family of runs of increasing model size that share data, tokenizer and a recipe for batch size,
duration, optimizer and learning-rate schedule (package of src/olmo_core/model_ladder/__init__.py).
"""

from .base import DeviceMeshSpec, ModelConfigurator, ModelLadder, RunCheckpointInfo, RunConfigurator
from .transformer_model_configurator import Olmo3ModelConfigurator, TransformerModelConfigurator, TransformerSize
from .wsds_chinchilla_run_configurator import WSDSChinchillaRunConfigurator

__all__ = ["ModelLadder", "ModelConfigurator", "RunConfigurator", "RunCheckpointInfo", "DeviceMeshSpec",
           "WSDSChinchillaRunConfigurator", "TransformerModelConfigurator", "Olmo3ModelConfigurator", "TransformerSize"]
