"""Optimizers and learning-rate schedulers (src/olmo_core/optim/__init__.py:32-66)."""

from .adam import AdamConfig
from .adamw import AdamWConfig, SkipStepAdamW, SkipStepAdamWConfig
from .config import INITIAL_LR_FIELD, LR_FIELD, MatrixAwareOptimConfig, OptimConfig, OptimGroupOverride
from .dion import DionConfig
from .lion import Lion, LionConfig, SkipStepLion, SkipStepLionConfig
from .muon import MuonConfig, NorMuonConfig
from .noop import NoOpConfig, NoOpOptimizer
from .scheduler import (
    ComposableScheduler, ConstantScheduler, ConstantWithWarmup, CosWithWarmup, CosWithWarmupAndLinearDecay,
    ExponentialScheduler, HalfCosWithWarmup, InvSqrtWithWarmup, LinearWithWarmup, PowerLR, Scheduler,
    SchedulerUnits, SequentialScheduler, WSD, WSDS,
)
from .skip_step_optimizer import SkipStepOptimizer

__all__ = [
    "AdamConfig", "AdamWConfig", "ComposableScheduler", "ConstantScheduler", "ConstantWithWarmup",
    "CosWithWarmup", "CosWithWarmupAndLinearDecay", "DionConfig", "ExponentialScheduler", "HalfCosWithWarmup",
    "INITIAL_LR_FIELD", "InvSqrtWithWarmup", "LR_FIELD", "LinearWithWarmup", "Lion", "LionConfig",
    "MatrixAwareOptimConfig", "MuonConfig", "NoOpConfig", "NoOpOptimizer", "NorMuonConfig", "OptimConfig",
    "OptimGroupOverride", "PowerLR", "Scheduler", "SchedulerUnits", "SequentialScheduler", "SkipStepAdamW",
    "SkipStepAdamWConfig", "SkipStepLion", "SkipStepLionConfig", "SkipStepOptimizer", "WSD", "WSDS",
]
