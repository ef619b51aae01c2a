"""Training loop, train modules, callbacks and checkpointing."""

from .common import Duration, DurationUnit, LoadStrategy, MetricMergeStrategy, ReduceType, StepSkipRange

__all__ = ["Duration", "DurationUnit", "LoadStrategy", "MetricMergeStrategy", "ReduceType", "StepSkipRange"]
