"""
Token permutation primitives of the mixture-of-experts layers under the names of src/olmo_core/kernels/moe.py:104-536.
The implementations live in :mod:`olmo_core_b200.ops.moe` (CUDA kernels on a GPU, index arithmetic on CPU); this module
only adapts the positional signatures.

Conventions: ``x [tokens, d]``; ``indices [tokens * top_k]`` is the argsort of the flattened expert assignment, so entry
``i`` of the permuted layout reads token ``indices[i] // top_k``; ``bin_ids`` is the sorted expert id per entry and
``bins`` the inclusive prefix sum of tokens per expert.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import moe as _ops

__all__ = ["gather", "scatter", "padded_scatter", "scatter_wgrad", "padded_scatter_wgrad", "binned_gather",
           "binned_scatter", "binned_scatter_wgrad"]


def gather(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, weights: Optional[torch.Tensor],
           bins: torch.Tensor, top_k: int) -> torch.Tensor:
    out = _ops.gather(x, indices, bin_ids, bins, top_k)
    if weights is not None:
        out = out * weights[indices].unsqueeze(-1).to(out.dtype)
    return out


def padded_scatter(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, weights: Optional[torch.Tensor],
                   bins: torch.Tensor, padded_bins: torch.Tensor, top_k: int) -> torch.Tensor:
    """``x`` holds each expert's rows starting at its padded offset; rows are compacted before the weighted scatter."""
    if padded_bins is not bins and not torch.equal(padded_bins, bins):
        starts = torch.cat([bins.new_zeros(1), bins[:-1]])
        padded_starts = torch.cat([padded_bins.new_zeros(1), padded_bins[:-1]])
        entry = torch.arange(indices.numel(), device=x.device)
        x = x[(padded_starts[bin_ids.long()] + entry - starts[bin_ids.long()]).long()]
    return _ops.scatter(x, indices, bin_ids, weights, bins, top_k)


def scatter(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, weights: Optional[torch.Tensor],
            bins: torch.Tensor, top_k: int) -> torch.Tensor:
    return _ops.scatter(x, indices, bin_ids, weights, bins, top_k)


def padded_scatter_wgrad(x: torch.Tensor, grad: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor,
                         bins: torch.Tensor, padded_bins: torch.Tensor, top_k: int) -> torch.Tensor:
    """Gradient of the scatter with respect to the routing weights: one dot product per (token, slot)."""
    if padded_bins is not bins and not torch.equal(padded_bins, bins):
        starts = torch.cat([bins.new_zeros(1), bins[:-1]])
        padded_starts = torch.cat([padded_bins.new_zeros(1), padded_bins[:-1]])
        entry = torch.arange(indices.numel(), device=x.device)
        x = x[(padded_starts[bin_ids.long()] + entry - starts[bin_ids.long()]).long()]
    dots = (x.float() * grad[(indices // top_k).long()].float()).sum(dim=-1)
    out = torch.empty_like(dots)
    out[indices.long()] = dots
    return out.to(x.dtype)


def scatter_wgrad(x: torch.Tensor, grad: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, bins: torch.Tensor,
                  top_k: int) -> torch.Tensor:
    return padded_scatter_wgrad(x, grad, indices, bin_ids, bins, bins, top_k)


def binned_gather(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], bins: torch.Tensor,
                  expert_capacity: int, top_k: int) -> torch.Tensor:
    out = _ops.binned_gather(x, indices, bins, expert_capacity, top_k)
    if weights is not None:
        raise NotImplementedError("weighted binned gather is not used by any layer")
    return out


def binned_scatter(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], bins: torch.Tensor,
                   top_k: int) -> torch.Tensor:
    return _ops.binned_scatter(x, indices, weights, bins, top_k)


def binned_scatter_wgrad(x: torch.Tensor, grad: torch.Tensor, indices: torch.Tensor, bins: torch.Tensor,
                         top_k: int) -> torch.Tensor:
    """``x [experts, capacity, d]``; returns the gradient of the routing weights, zero for dropped entries."""
    E, cap, _ = x.shape
    starts = torch.cat([bins.new_zeros(1), bins[:-1]]).long()
    out = torch.zeros(indices.numel(), dtype=torch.float32, device=x.device)
    for e in range(E):
        n = min(int(bins[e]) - int(starts[e]), cap)
        if n <= 0:
            continue
        entries = indices[starts[e]:starts[e] + n].long()
        out[entries] = (x[e, :n].float() * grad[entries // top_k].float()).sum(-1)
    return out.to(x.dtype)


def assert_is_tensor(x, ndim):
    if x.ndim != ndim:
        raise ValueError(f"Expected {ndim}-tensor but got {x.ndim}-tensor")


def assert_is_matrix(x):
    assert_is_tensor(x, 2)


def assert_is_vector(x):
    assert_is_tensor(x, 1)


def assert_equal(a, b):
    if a != b:
        raise ValueError(f"Expected dimensions to be equal but got {a} and {b}.")
