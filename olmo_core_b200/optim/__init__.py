"""Optimizers and learning-rate schedulers (src/olmo_core/optim/__init__.py:32-66)."""

from .adam import AdamConfig
from .adamw import AdamWConfig, SkipStepAdamW, SkipStepAdamWConfig
from .config import INITIAL_LR_FIELD, LR_FIELD, MatrixAwareOptimConfig, OptimConfig, OptimGroupOverride
from .dion import DionConfig
from .lion import Lion, LionConfig, SkipStepLion, SkipStepLionConfig
from .muon import MuonConfig, NorMuonConfig
from .noop import NoOpConfig, NoOpOptimizer
from .scheduler import (
    WSD,
    WSDS,
    ComposableScheduler,
    ConstantScheduler,
    ConstantWithWarmup,
    CosWithWarmup,
    CosWithWarmupAndLinearDecay,
    ExponentialScheduler,
    HalfCosWithWarmup,
    InvSqrtWithWarmup,
    LinearWithWarmup,
    PowerLR,
    Scheduler,
    SchedulerUnits,
    SequentialScheduler,
)
from .skip_step_optimizer import SkipStepOptimizer

__all__ = [
    "OptimConfig",
    "MatrixAwareOptimConfig",
    "OptimGroupOverride",
    "SkipStepOptimizer",
    "AdamWConfig",
    "SkipStepAdamWConfig",
    "SkipStepAdamW",
    "AdamConfig",
    "LionConfig",
    "Lion",
    "MuonConfig",
    "NorMuonConfig",
    "DionConfig",
    "SkipStepLionConfig",
    "SkipStepLion",
    "NoOpConfig",
    "NoOpOptimizer",
    "Scheduler",
    "SchedulerUnits",
    "ConstantScheduler",
    "ConstantWithWarmup",
    "CosWithWarmup",
    "CosWithWarmupAndLinearDecay",
    "ComposableScheduler",
    "ExponentialScheduler",
    "HalfCosWithWarmup",
    "InvSqrtWithWarmup",
    "LinearWithWarmup",
    "SequentialScheduler",
    "WSD",
    "WSDS",
    "PowerLR",
    "LR_FIELD",
    "INITIAL_LR_FIELD",
]
