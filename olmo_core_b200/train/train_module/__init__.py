"""Train modules (src/olmo_core/train/train_module/__init__.py:23)."""

from .config import TrainModuleConfig
from .train_module import BasicTrainModule, EvalBatchSizeUnit, EvalBatchSpec, TrainModule
from .transformer import (
    TransformerActivationCheckpointingConfig, TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig, TransformerDataParallelConfig, TransformerDataParallelWrappingStrategy,
    TransformerExpertParallelConfig, TransformerPipelineParallelConfig, TransformerPipelineTrainModule,
    TransformerPipelineTrainModuleConfig, TransformerTensorParallelConfig, TransformerTrainModule,
    TransformerTrainModuleConfig,
)

__all__ = [
    "BasicTrainModule", "EvalBatchSizeUnit", "EvalBatchSpec", "TrainModule", "TrainModuleConfig",
    "TransformerActivationCheckpointingConfig", "TransformerActivationCheckpointingMode",
    "TransformerContextParallelConfig", "TransformerDataParallelConfig",
    "TransformerDataParallelWrappingStrategy", "TransformerExpertParallelConfig",
    "TransformerPipelineParallelConfig", "TransformerPipelineTrainModule", "TransformerPipelineTrainModuleConfig",
    "TransformerTensorParallelConfig", "TransformerTrainModule", "TransformerTrainModuleConfig",
]
