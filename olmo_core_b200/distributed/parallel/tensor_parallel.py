"""Tensor-parallel configuration (src/olmo_core/distributed/parallel/tensor_parallel.py:17-40)."""

from dataclasses import dataclass

from ...config import Config

__all__ = ["TensorParallelConfig", "SequenceParallel"]


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


def __getattr__(name: str):
    # ``SequenceParallel`` (src/olmo_core/distributed/parallel/tensor_parallel.py:43-68): the DTensor parallel style whose
    # output placement can be chosen. Built on first use so that importing this module does not pull in DTensor.
    if name == "SequenceParallel":
        from functools import partial

        import torch.nn as nn
        from torch.distributed.tensor import Shard, distribute_module
        from torch.distributed.tensor.parallel import SequenceParallel as _Base

        class SequenceParallel(_Base):
            """Replicated module over sequence-sharded activations; ``output_layouts`` (default: sharded on the sequence
            dimension) says how the output is left."""

            def __init__(self, *, sequence_dim: int = 1, use_local_output: bool = False, output_layouts=None):
                super().__init__(sequence_dim=sequence_dim, use_local_output=use_local_output)
                self.output_layouts = (output_layouts or Shard(sequence_dim),)

            @staticmethod
            def _prepare_output_fn(output_layouts, use_local_output, mod, outputs, device_mesh):
                if outputs.placements != output_layouts:
                    outputs = outputs.redistribute(placements=output_layouts, async_op=True)
                return outputs.to_local() if use_local_output else outputs

            def _apply(self, module: nn.Module, device_mesh) -> nn.Module:
                return distribute_module(
                    module, device_mesh, self._replicate_module_fn,
                    partial(self._prepare_input_fn, self.sequence_sharding),
                    partial(self._prepare_output_fn, self.output_layouts, self.use_local_output))

        globals()["SequenceParallel"] = SequenceParallel
        return SequenceParallel
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
