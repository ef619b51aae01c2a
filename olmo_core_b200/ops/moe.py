"""
Token permutation ops for mixture-of-experts layers (function names of src/olmo_core/ops/moe.py:52-304,
whose reference implementation is a set of Triton copy kernels, src/olmo_core/kernels/moe.py:31-536).

Layout conventions: ``top_experts`` is ``[N, k]``; flattening it gives ``N*k`` routed copies. Sorting the
flat list by expert id (stable) gives ``indices`` (positions in the flat list, so token = index // k) and
``bins`` (inclusive cumulative sum of tokens per expert). ``gather`` builds the expert-sorted activation
matrix, ``scatter`` is its inverse and applies the router weights, summing the ``k`` copies of each token
in fp32.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

__all__ = [
    "indices_and_bins",
    "gather",
    "scatter",
    "binned_gather",
    "binned_scatter",
    "histc",
    "batched_histc",
    "repeat",
    "sum_tensor",
    "all_to_all",
    "GatherOp",
    "ScatterOp",
    "BinnedGatherOp",
    "BinnedScatterOp",
    "AllToAllOp",
]


def histc(x: torch.Tensor, num_classes: int) -> torch.Tensor:
    """Count occurrences of each id in ``[0, num_classes)`` (int64 result, any input shape)."""
    return torch.bincount(x.reshape(-1), minlength=num_classes)[:num_classes]


def batched_histc(x: torch.Tensor, num_classes: int) -> torch.Tensor:
    """Histogram over the last dimension: ``[..., k] -> [..., num_classes]``."""
    out = torch.zeros(*x.shape[:-1], num_classes, dtype=x.dtype, device=x.device)
    out.scatter_add_(-1, x, torch.ones_like(x))
    return out


def _use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and t.stride(1) == 1


def _inverse(indices: torch.Tensor) -> torch.Tensor:
    """``dest`` with ``dest[indices[r]] = r``: the row of every routed copy (cached on the tensor by ``indices_and_bins``)."""
    dest = getattr(indices, "_dest", None)
    if dest is None:
        dest = torch.empty_like(indices)
        dest[indices.long()] = torch.arange(indices.numel(), device=indices.device, dtype=indices.dtype)
    return dest


@torch.no_grad()
def indices_and_bins(top_experts: torch.Tensor, num_experts: int,
                     counts: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    Returns ``(indices, bin_ids, bins)``: the stable sort permutation of the flattened expert ids, the
    sorted ids themselves, and the inclusive cumulative token count per expert (all int32).

    On CUDA this is one counting sort (three small kernels, no host synchronisation). The inverse permutation and the
    exclusive offsets ``[E + 1]`` that the grouped GEMM consumes ride along as ``indices._dest`` / ``bins._offsets``.
    """
    flat = top_experts.reshape(-1)
    if flat.is_cuda and num_experts <= 1024:
        from . import _lib

        n = flat.numel()
        experts = flat if flat.dtype == torch.int32 else flat.to(torch.int32)
        dest = torch.empty(n, dtype=torch.int32, device=flat.device)
        src = torch.empty_like(dest)
        bin_ids = torch.empty_like(dest)
        offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=flat.device)
        scratch = torch.empty(n + ((n + 2047) // 2048) * num_experts, dtype=torch.int32, device=flat.device)
        rc = _lib.lib().ocb_moe_sort(experts.data_ptr(), dest.data_ptr(), src.data_ptr(), bin_ids.data_ptr(),
                                     offsets.data_ptr(), scratch.data_ptr(), n, num_experts, _lib.stream_ptr())
        _lib.check(rc, "ocb_moe_sort")
        bins = offsets[1:]
        src._dest = dest  # type: ignore[attr-defined]
        bins._offsets = offsets  # type: ignore[attr-defined]
        return src, bin_ids, bins
    bin_ids, indices = torch.sort(flat, stable=True)
    if counts is None:
        counts = histc(flat, num_experts)
    bins = torch.cumsum(counts, 0)
    return indices.to(torch.int32), bin_ids.to(torch.int32), bins.to(torch.int32)


def _gather_rows(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], top_k: int) -> torch.Tensor:
    from . import _lib

    out = torch.empty((indices.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    rc = _lib.lib().ocb_moe_gather(x.data_ptr(), indices.data_ptr(), _lib.ptr(weights), out.data_ptr(), indices.numel(),
                                   x.shape[1], top_k, x.stride(0), out.stride(0), _lib.stream_ptr())
    _lib.check(rc, "ocb_moe_gather")
    return out


def _scatter_rows(ys: torch.Tensor, dest: torch.Tensor, weights: Optional[torch.Tensor], top_k: int) -> torch.Tensor:
    from . import _lib

    n_tokens = dest.numel() // top_k
    out = torch.empty((n_tokens, ys.shape[1]), dtype=ys.dtype, device=ys.device)
    rc = _lib.lib().ocb_moe_scatter(ys.data_ptr(), dest.data_ptr(), _lib.ptr(weights), out.data_ptr(), n_tokens,
                                    ys.shape[1], top_k, ys.stride(0), out.stride(0), _lib.stream_ptr())
    _lib.check(rc, "ocb_moe_scatter")
    return out


def _flat_weights(weights: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if weights is None:
        return None
    w = weights.reshape(-1)
    return w.contiguous() if w.dtype == torch.float32 else w.float()


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices, top_k: int):  # type: ignore[override]
        ctx.n_tokens, ctx.top_k = x.shape[0], top_k
        if _use_kernels(x) and indices.dtype == torch.int32:
            ctx.kernel = True
            ctx.save_for_backward(_inverse(indices))
            return _gather_rows(x, indices, None, top_k)
        ctx.kernel = False
        tok = (indices // top_k).long()
        ctx.save_for_backward(tok)
        return x.index_select(0, tok)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        (saved,) = ctx.saved_tensors
        if ctx.kernel:  # the k copies of a token sum up: the same kernel as the forward scatter, without weights
            return _scatter_rows(grad.contiguous(), saved, None, ctx.top_k), None, None
        dx = torch.zeros((ctx.n_tokens, grad.shape[1]), dtype=torch.float32, device=grad.device)
        dx.index_add_(0, saved, grad.float())
        return dx.to(grad.dtype), None, None


def gather(x: torch.Tensor, indices: torch.Tensor, bin_ids: Optional[torch.Tensor], bins: Optional[torch.Tensor],
           top_k: int) -> torch.Tensor:
    """Expert-sorted copy of the tokens: ``out[i] = x[indices[i] // top_k]``; ``x`` is ``[N, d]``."""
    return _Gather.apply(x, indices, top_k)


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices, weights, top_k: int):  # type: ignore[override]
        ctx.top_k = top_k
        ctx.has_w = weights is not None
        if _use_kernels(x) and indices.dtype == torch.int32:
            ctx.kernel = True
            dest = _inverse(indices)
            w = _flat_weights(weights)
            ctx.save_for_backward(x, indices, dest, w if w is not None else torch.empty(0, device=x.device))
            ctx.w_meta = None if weights is None else (weights.shape, weights.dtype)
            return _scatter_rows(x, dest, w, top_k)
        ctx.kernel = False
        n_tokens = x.shape[0] // top_k
        idx = indices.long()
        w = None
        if weights is not None:
            w = weights.reshape(-1).index_select(0, idx).float()
        scaled = x.float() if w is None else x.float() * w[:, None]
        out = torch.zeros((n_tokens, x.shape[1]), dtype=torch.float32, device=x.device)
        out.index_add_(0, idx // top_k, scaled)
        ctx.save_for_backward(x, idx, weights if weights is not None else torch.empty(0, device=x.device))
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        if ctx.kernel:
            from . import _lib

            x, indices, dest, w = ctx.saved_tensors
            grad = grad.contiguous()
            dx = _gather_rows(grad, indices, w if ctx.has_w else None, ctx.top_k)
            dw = None
            if ctx.has_w and ctx.needs_input_grad[2]:
                shape, dtype = ctx.w_meta
                dwf = torch.empty(indices.numel(), dtype=torch.float32, device=x.device)
                rc = _lib.lib().ocb_moe_rowdot(x.data_ptr(), dest.data_ptr(), grad.data_ptr(), dwf.data_ptr(),
                                               indices.numel(), x.shape[1], ctx.top_k, x.stride(0), grad.stride(0),
                                               _lib.stream_ptr())
                _lib.check(rc, "ocb_moe_rowdot")
                dw = dwf.view(shape).to(dtype)
            return dx, None, dw, None
        x, idx, weights = ctx.saved_tensors
        g = grad.index_select(0, idx // ctx.top_k)  # gradient of each routed copy before weighting
        dx = g
        dw = None
        if ctx.has_w:
            w = weights.reshape(-1).index_select(0, idx)
            dx = (g.float() * w.float()[:, None]).to(x.dtype)
            if ctx.needs_input_grad[2]:
                per_copy = (g.float() * x.float()).sum(-1)
                dw = torch.zeros(weights.numel(), dtype=torch.float32, device=x.device)
                dw.index_copy_(0, idx, per_copy)
                dw = dw.view_as(weights).to(weights.dtype)
        return dx, None, dw, None


def scatter(x: torch.Tensor, indices: torch.Tensor, bin_ids: Optional[torch.Tensor], weights: Optional[torch.Tensor],
            bins: Optional[torch.Tensor], top_k: int) -> torch.Tensor:
    """Inverse of :func:`gather`: ``out[t] = sum_j weights[t, j] * x[position of copy (t, j)]`` in fp32."""
    return _Scatter.apply(x, indices, weights, top_k)


def binned_gather(x: torch.Tensor, indices: torch.Tensor, bins: torch.Tensor, bin_size: int, top_k: int) -> torch.Tensor:
    """
    Capacity-limited layout ``[num_experts, bin_size, d]``: the first ``bin_size`` tokens routed to each
    expert are copied, the rest are dropped, unused slots are zero.
    """
    capacity = bin_size
    E = bins.numel()
    pos = torch.arange(indices.numel(), device=x.device)
    starts = torch.cat([bins.new_zeros(1), bins[:-1]]).long()
    expert_of = torch.bucketize(pos, bins.long(), right=True).clamp(max=E - 1)
    slot = pos - starts[expert_of]
    keep = slot < capacity
    flat_dst = (expert_of * capacity + slot)[keep]
    src = (indices.long() // top_k)[keep]
    out = x.new_zeros((E * capacity, x.shape[1]))
    out = out.index_copy(0, flat_dst, x.index_select(0, src))
    return out.view(E, capacity, x.shape[1])


def binned_scatter(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], bins: torch.Tensor,
                   top_k: int) -> torch.Tensor:
    """Inverse of :func:`binned_gather` with router weights; dropped tokens contribute zero."""
    E, capacity, d = x.shape
    pos = torch.arange(indices.numel(), device=x.device)
    starts = torch.cat([bins.new_zeros(1), bins[:-1]]).long()
    expert_of = torch.bucketize(pos, bins.long(), right=True).clamp(max=E - 1)
    slot = pos - starts[expert_of]
    keep = slot < capacity
    flat_src = (expert_of * capacity + slot)[keep]
    idx = indices.long()[keep]
    rows = x.reshape(E * capacity, d).index_select(0, flat_src).float()
    if weights is not None:
        rows = rows * weights.reshape(-1).index_select(0, idx).float()[:, None]
    n_tokens = indices.numel() // top_k
    out = torch.zeros((n_tokens, d), dtype=torch.float32, device=x.device)
    out = out.index_add(0, idx // top_k, rows)
    return out.to(x.dtype)


def repeat(x: torch.Tensor, tiling) -> torch.Tensor:
    if all(t == 1 for t in tiling):
        return x
    return x.repeat(*tiling)


def sum_tensor(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return x.squeeze(dim) if x.shape[dim] == 1 else x.sum(dim=dim)


class _AllToAllAsync(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, output_split_sizes, input_split_sizes, group, async_op: bool):  # type: ignore[override]
        out_rows = x.shape[0] if output_split_sizes is None else sum(output_split_sizes)
        out = x.new_empty((out_rows,) + tuple(x.shape[1:]))
        ctx.splits = (output_split_sizes, input_split_sizes)
        ctx.group = group
        ctx.in_shape = x.shape
        handle = dist.all_to_all_single(out, x.contiguous(), output_split_sizes=output_split_sizes,
                                        input_split_sizes=input_split_sizes, group=group, async_op=async_op)
        ctx.mark_non_differentiable()
        return out, handle

    @staticmethod
    def backward(ctx, grad, _):  # type: ignore[override]
        out_splits, in_splits = ctx.splits
        back = grad.new_empty(ctx.in_shape)
        dist.all_to_all_single(back, grad.contiguous(), output_split_sizes=in_splits, input_split_sizes=out_splits,
                               group=ctx.group)
        return back, None, None, None, None


def all_to_all(x: torch.Tensor, output_split_sizes=None, input_split_sizes=None, group=None, async_op: bool = False):
    """Row exchange with variable split sizes; returns ``(output, work handle or None)``."""
    return _AllToAllAsync.apply(x, output_split_sizes, input_split_sizes, group, async_op)


class _OpNamespace:
    """``Name.apply(...)`` spelling of an op, for code written against the autograd-function classes of
    src/olmo_core/ops/moe.py (``GatherOp``, ``ScatterOp``, ``BinnedGatherOp``, ``BinnedScatterOp``, ``AllToAllOp``)."""

    _fn = None

    @classmethod
    def apply(cls, *args):
        return cls._fn(*args)


class GatherOp(_OpNamespace):
    """``apply(x, indices, bin_ids, bins, top_k)``"""

    _fn = staticmethod(gather)


class ScatterOp(_OpNamespace):
    """``apply(x, indices, bin_ids, weights, bins, top_k)``"""

    _fn = staticmethod(scatter)


class BinnedGatherOp(_OpNamespace):
    """``apply(x, indices, bins, bin_size, top_k)``"""

    _fn = staticmethod(binned_gather)


class BinnedScatterOp(_OpNamespace):
    """``apply(x, indices, weights, bins, top_k)``"""

    _fn = staticmethod(binned_scatter)


AllToAllOp = _AllToAllAsync
