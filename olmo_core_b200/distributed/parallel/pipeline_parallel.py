"""
Pipeline-parallel configuration and schedule wrapper
(src/olmo_core/distributed/parallel/pipeline_parallel.py:20-221). Stage send/recv stays on NCCL
point-to-point through ``torch.distributed.pipelining``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from ...config import Config, StrEnum
from ...exceptions import OLMoConfigurationError

__all__ = ["PipelineSplitStyle", "PipelineScheduleType", "PipelineParallelConfig", "PipelineSchedule"]


class PipelineSplitStyle(StrEnum):
    loop = "loop"
    v = "v"


class PipelineScheduleType(StrEnum):
    single_1F1B = "1F1B"
    interleaved_1F1B = "Interleaved1F1B"
    gpipe = "GPipe"
    looped_bfs = "LoopedBFS"
    interleaved_zero_bubble = "InterleavedZeroBubble"
    zbv_zero_bubble = "ZBVZeroBubble"
    custom_1F1B = "custom_1F1B"
    custom_interleaved_1F1B = "custom_interleaved_1F1B"

    @property
    def is_single_stage(self) -> bool:
        return self in (PipelineScheduleType.single_1F1B, PipelineScheduleType.gpipe, PipelineScheduleType.custom_1F1B)

    @property
    def is_multi_stage(self) -> bool:
        return not self.is_single_stage

    @property
    def default_style(self) -> PipelineSplitStyle:
        return PipelineSplitStyle.v if self == PipelineScheduleType.zbv_zero_bubble else PipelineSplitStyle.loop


@dataclass
class PipelineParallelConfig(Config):
    degree: int
    schedule: PipelineScheduleType = PipelineScheduleType.single_1F1B
    style: Optional[PipelineSplitStyle] = None

    def __post_init__(self):
        self.schedule = PipelineScheduleType(self.schedule)
        if self.style is not None:
            self.style = PipelineSplitStyle(self.style)

    def infer_style(self) -> PipelineSplitStyle:
        return self.style or self.schedule.default_style

    def final_stage_rank(self) -> int:
        """PP rank that holds the last stage (rank 0 for the V layout, the last rank for loops)."""
        return 0 if self.infer_style() == PipelineSplitStyle.v else self.degree - 1

    def rank_completion_order(self) -> Iterable[int]:
        """Order in which PP ranks finish a step, starting from the rank with the last stage."""
        if self.infer_style() == PipelineSplitStyle.v:
            return range(self.degree)
        return range(self.degree - 1, -1, -1)

    def stage_ids_this_rank(self, pp_rank: int, num_stages: int) -> Tuple[int, ...]:
        if num_stages % self.degree != 0:
            raise OLMoConfigurationError(f"num_stages ({num_stages}) must be a multiple of the PP degree ({self.degree})")
        per_rank = num_stages // self.degree
        style = self.infer_style()
        if style == PipelineSplitStyle.loop:
            return tuple(pp_rank + s * self.degree for s in range(per_rank))
        if per_rank != 2:
            raise OLMoConfigurationError("the 'v' layout needs exactly two stages per rank")
        return (pp_rank, num_stages - 1 - pp_rank)


class PipelineSchedule:
    """Thin wrapper that builds a ``torch.distributed.pipelining`` schedule for a list of local stages."""

    def __init__(self, *, model_parts: List[nn.Module], stages: List[Any], pp_mesh, schedule_name: PipelineScheduleType,
                 loss_fn: Optional[Callable[[Any, torch.Tensor], torch.Tensor]] = None, num_microbatches: Optional[int] = None):
        from torch.distributed.pipelining.schedules import (
            PipelineScheduleMulti,
            PipelineScheduleSingle,
            get_schedule_class,
        )

        self.model_parts = model_parts
        self.stages = stages
        self.pp_mesh = pp_mesh
        self.loss_fn = loss_fn
        pp_size = pp_mesh.size()
        n_mb = num_microbatches if num_microbatches is not None else pp_size
        name = {"custom_1F1B": "1F1B", "custom_interleaved_1F1B": "Interleaved1F1B"}.get(schedule_name.value, schedule_name.value)
        cls = get_schedule_class(name)
        if issubclass(cls, PipelineScheduleSingle):
            if len(stages) != 1:
                raise OLMoConfigurationError(f"schedule {name} takes exactly one stage per rank")
            self.base_schedule = cls(stages[0], n_microbatches=n_mb, loss_fn=loss_fn)
        else:
            assert issubclass(cls, PipelineScheduleMulti)
            self.base_schedule = cls(stages, n_microbatches=n_mb, loss_fn=loss_fn)
        self.num_microbatches = n_mb

    @property
    def is_first_stage(self) -> bool:
        return any(s.is_first for s in self.stages)

    @property
    def is_last_stage(self) -> bool:
        return any(s.is_last for s in self.stages)

    has_first_stage = is_first_stage
    has_last_stage = is_last_stage

    def step(self, *args, target: Optional[torch.Tensor] = None, **kwargs) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """Run one pipelined forward/backward. Returns (output of the last stage, summed loss) where held."""
        losses: List[torch.Tensor] = []
        if self.is_first_stage:
            out = self.base_schedule.step(*args, target=target if self.is_last_stage else None,
                                          losses=losses if self.is_last_stage else None, **kwargs)
        else:
            out = self.base_schedule.step(target=target if self.is_last_stage else None,
                                          losses=losses if self.is_last_stage else None, **kwargs)
        loss = torch.stack(losses).sum() if losses else None
        return out, loss
