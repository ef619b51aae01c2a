"""Tensor-parallel configuration (src/olmo_core/distributed/parallel/tensor_parallel.py:17-40)."""

from dataclasses import dataclass

from ...config import Config

__all__ = ["TensorParallelConfig"]


@dataclass
class TensorParallelConfig(Config):
    """
    ``degree``-way tensor parallelism with sequence-parallel norms/residuals. ``enable_async`` selects the
    fused all-gather->GEMM / GEMM->reduce-scatter kernels over peer memory instead of separate
    collectives followed by GEMMs.
    """

    degree: int
    enable_async: bool = False

    def maybe_enable_async_tp(self, tp_mesh) -> None:
        if self.enable_async:
            from ...parallel.symmetric import ensure_symmetric_group

            ensure_symmetric_group(tp_mesh.get_group())
