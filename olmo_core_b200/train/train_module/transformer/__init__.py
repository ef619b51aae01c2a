from .config import (
    TransformerActivationCheckpointingConfig,
    TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig,
    TransformerDataParallelConfig,
    TransformerDataParallelWrappingStrategy,
    TransformerExpertParallelConfig,
    TransformerPipelineParallelConfig,
    TransformerPipelineTrainModuleConfig,
    TransformerTensorParallelConfig,
    TransformerTrainModuleConfig,
)
from .pipeline_train_module import TransformerPipelineTrainModule
from .train_module import TransformerTrainModule

__all__ = [
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
