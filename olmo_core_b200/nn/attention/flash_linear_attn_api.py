"""
Entry points for the linear-attention primitives (names of src/olmo_core/nn/attention/flash_linear_attn_api.py:11-63),
served by this package's own implementations rather than an external library.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

__all__ = ["has_fla", "dispatch_chunk_gated_delta_rule", "dispatch_causal_conv1d"]


def has_fla() -> bool:
    """Always true: the chunked gated delta rule and the causal convolution are built in."""
    return True


def dispatch_chunk_gated_delta_rule(q, k, v, g, beta, scale: Optional[float] = None, initial_state=None,
                                    output_final_state: bool = False, use_qk_l2norm_in_kernel: bool = False,
                                    cu_seqlens=None):
    """``q, k: [B, T, H, Dk]``, ``v: [B, T, H, Dv]``, ``g, beta: [B, T, H]``; returns ``(out, final_state | None)``."""
    from .recurrent import gated_delta_rule

    if initial_state is not None or output_final_state:
        raise NotImplementedError("carrying recurrent state across calls is not supported by the chunked form")
    if use_qk_l2norm_in_kernel:
        q, k = F.normalize(q.float(), dim=-1).to(q.dtype), F.normalize(k.float(), dim=-1).to(k.dtype)
    if cu_seqlens is None:
        return gated_delta_rule(q, k, v, g, beta, scale=scale), None
    # packed documents ([1, total, ...]): the state must not leak across boundaries, so each document runs alone
    bounds = cu_seqlens.tolist()
    pieces = [gated_delta_rule(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b], scale=scale)
              for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
    return torch.cat(pieces, dim=1), None


def dispatch_causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation: Optional[str],
                           backend: str = "cuda", cu_seqlens=None) -> torch.Tensor:
    """Depth-wise causal convolution over ``x: [B, T, C]`` with ``weight: [C, K]``; optional SiLU."""
    del backend
    if activation not in (None, "silu", "swish"):
        raise ValueError(f"unsupported activation '{activation}'")

    def run(seg: torch.Tensor) -> torch.Tensor:
        k = weight.shape[-1]
        y = F.conv1d(F.pad(seg.transpose(1, 2), (k - 1, 0)), weight.unsqueeze(1), bias, groups=weight.shape[0])
        y = y.transpose(1, 2)
        return F.silu(y) if activation else y

    if cu_seqlens is None:
        return run(x)
    bounds = cu_seqlens.tolist()
    return torch.cat([run(x[:, a:b]) for a, b in zip(bounds[:-1], bounds[1:]) if b > a], dim=1)
