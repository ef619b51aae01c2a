"""Expert-parallel configuration (src/olmo_core/distributed/parallel/expert_parallel.py:6-15)."""

from dataclasses import dataclass

from ...config import Config

__all__ = ["ExpertParallelConfig"]


@dataclass
class ExpertParallelConfig(Config):
    """Experts of every MoE layer are split over ``degree`` ranks (-1: the whole shard group)."""

    degree: int = -1
