"""
Differentiable all-to-all primitives (src/olmo_core/distributed/nn.py:5-67): the backward of an
all-to-all is the all-to-all with the split sizes swapped.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

__all__ = ["all_to_all_single", "all_to_all"]


class _AllToAllSingle(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, output_split_sizes, input_split_sizes):  # type: ignore[override]
        ctx.group = group
        ctx.in_splits = input_split_sizes
        ctx.out_splits = output_split_sizes
        x = x.contiguous()
        if output_split_sizes is None:
            out = torch.empty_like(x)
        else:
            out = x.new_empty((sum(output_split_sizes),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes, input_split_sizes, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        g = _AllToAllSingle.apply(ctx.group, grad, ctx.in_splits, ctx.out_splits)
        return None, g, None, None


def all_to_all_single(
    group: Optional[dist.ProcessGroup],
    input_: torch.Tensor,
    output_split_sizes: Optional[Sequence[int]] = None,
    input_split_sizes: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Exchange slices of dim 0 of ``input_`` between the ranks of ``group`` (autograd-aware)."""
    x = input_
    outs = list(output_split_sizes) if output_split_sizes is not None else None
    ins = list(input_split_sizes) if input_split_sizes is not None else None
    return _AllToAllSingle.apply(group, x, outs, ins)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, out_like, *tensors):  # type: ignore[override]
        ctx.group = group
        ctx.in_shapes = [t.shape for t in tensors]
        outs = [torch.empty_like(o) for o in out_like]
        dist.all_to_all(outs, [t.contiguous() for t in tensors], group=group)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):  # type: ignore[override]
        like = [grads[0].new_empty(s) for s in ctx.in_shapes]
        back = _AllToAll.apply(ctx.group, like, *grads)
        return (None, None) + tuple(back)


def all_to_all(group: Optional[dist.ProcessGroup], input_tensor_list: List[torch.Tensor],
               output_like: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
    """List form: ``input_tensor_list[i]`` goes to rank ``i``; returns what each rank sent to us."""
    tensors = input_tensor_list
    output_like = output_like if output_like is not None else tensors
    return list(_AllToAll.apply(group, output_like, *tensors))
