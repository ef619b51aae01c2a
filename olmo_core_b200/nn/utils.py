"""Activation-checkpointing policy helpers (src/olmo_core/nn/utils.py)."""

from __future__ import annotations

from collections import defaultdict
from typing import Dict

import torch

__all__ = ["selective_checkpointing_context_fn", "get_tp_wrappers"]

# Outputs of these ops are kept; everything cheaper is recomputed in backward.
_SAVE_OPS = {"mm", "addmm", "bmm", "_scaled_dot_product_flash_attention", "_scaled_dot_product_efficient_attention",
             "_scaled_dot_product_cudnn_attention", "all_to_all_single", "reduce_scatter_tensor"}


def _op_name(func) -> str:
    return getattr(func, "__name__", str(func)).split(".")[0]


def selective_checkpointing_context_fn():
    """Context factory for ``torch.utils.checkpoint``: save GEMM / attention / collective outputs, every second matmul only."""
    from torch.utils.checkpoint import CheckpointPolicy, create_selective_checkpoint_contexts

    counts: Dict[str, int] = defaultdict(int)

    def policy(ctx, func, *args, **kwargs):
        name = _op_name(func)
        if name not in _SAVE_OPS:
            return CheckpointPolicy.PREFER_RECOMPUTE
        if name == "mm":
            key = "recompute_mm" if ctx.is_recompute else "forward_mm"
            counts[key] += 1
            if counts[key] % 2 == 0:
                return CheckpointPolicy.PREFER_RECOMPUTE
        return CheckpointPolicy.MUST_SAVE

    return create_selective_checkpoint_contexts(policy)


def get_tp_wrappers(float8_enabled: bool):
    """Kept for API compatibility: tensor parallelism here slices parameters in place (``parallel.tensor``)."""
    del float8_enabled
    from torch.distributed.tensor.parallel import ColwiseParallel, PrepareModuleInput, RowwiseParallel

    return RowwiseParallel, ColwiseParallel, PrepareModuleInput
