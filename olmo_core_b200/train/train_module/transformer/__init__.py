from .config import (
    TransformerActivationCheckpointingConfig, TransformerActivationCheckpointingMode,
    TransformerContextParallelConfig, TransformerDataParallelConfig, TransformerDataParallelWrappingStrategy,
    TransformerExpertParallelConfig, TransformerPipelineParallelConfig, TransformerPipelineTrainModuleConfig,
    TransformerTensorParallelConfig, TransformerTrainModuleConfig,
)
from .pipeline_train_module import TransformerPipelineTrainModule
from .train_module import TransformerTrainModule

__all__ = [
    "TransformerActivationCheckpointingConfig", "TransformerActivationCheckpointingMode",
    "TransformerContextParallelConfig", "TransformerDataParallelConfig",
    "TransformerDataParallelWrappingStrategy", "TransformerExpertParallelConfig",
    "TransformerPipelineParallelConfig", "TransformerPipelineTrainModule", "TransformerPipelineTrainModuleConfig",
    "TransformerTensorParallelConfig", "TransformerTrainModule", "TransformerTrainModuleConfig",
]
