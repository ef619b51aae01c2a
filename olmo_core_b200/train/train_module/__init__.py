"""Train modules (src/olmo_core/train/train_module/__init__.py:23)."""

from .config import TrainModuleConfig
from .train_module import BasicTrainModule, EvalBatchSizeUnit, EvalBatchSpec, TrainModule
from .transformer import (
    TransformerActivationCheckpointingConfig,
    TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig,
    TransformerDataParallelConfig,
    TransformerDataParallelWrappingStrategy,
    TransformerExpertParallelConfig,
    TransformerPipelineParallelConfig,
    TransformerPipelineTrainModuleConfig,
    TransformerPipelineTrainModule,
    TransformerTensorParallelConfig,
    TransformerTrainModule,
    TransformerTrainModuleConfig,
)

__all__ = [
    "TrainModuleConfig",
    "TrainModule",
    "EvalBatchSpec",
    "EvalBatchSizeUnit",
    "BasicTrainModule",
    "TransformerTrainModule",
    "TransformerTrainModuleConfig",
    "TransformerPipelineTrainModule",
    "TransformerPipelineTrainModuleConfig",
    "TransformerActivationCheckpointingConfig",
    "TransformerActivationCheckpointingMode",
    "TransformerDataParallelConfig",
    "TransformerDataParallelWrappingStrategy",
    "TransformerExpertParallelConfig",
    "TransformerTensorParallelConfig",
    "TransformerContextParallelConfig",
    "TransformerPipelineParallelConfig",
]
