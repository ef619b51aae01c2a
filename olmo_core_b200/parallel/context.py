"""
Context-parallel attention over a sequence that is sharded across a process group
(role of the ring-flash-attn / all-gather-KV paths in src/olmo_core/nn/attention/backend.py:446-640 and
src/olmo_core/nn/attention/ring.py).

Each rank holds the queries, keys and values of its own sequence shard -- contiguous for the ``llama3`` layout, two
mirrored chunks (``r`` and ``2*cp-1-r``) for the load-balanced ``zig_zag`` layout. Keys and values are all-gathered over
the group (autograd-aware: the backward pass reduce-scatters their gradients) and put into global order; every local
query chunk, being a contiguous range of global positions ``[a, b)``, then runs ordinary causal attention against keys
``[0, b)`` aligned at the end. Compared with a ring exchange this trades ``cp``-times more resident K/V (small next to
180 GB: 2 x T x Hkv x D x 2 bytes per layer) for a single collective per layer and one attention call per chunk.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["ring_attention", "local_position_ranges"]


class _AllGatherSeq(torch.autograd.Function):
    """``[B, T_local, ...] -> [cp, B, T_local, ...]``; backward sums the gradient slices back onto their owners."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        ws = dist.get_world_size(group)
        out = torch.empty((ws,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out.view(-1), x.contiguous().view(-1), group=group)
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        group = ctx.group
        ws, rank = dist.get_world_size(group), dist.get_rank(group)
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty_like(g[0])
            dist.reduce_scatter_tensor(out.view(-1), g.view(-1), op=dist.ReduceOp.SUM, group=group)
        else:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
            out = g[rank].clone()
        return out, None


def local_position_ranges(local_len: int, rank: int, cp: int, zig_zag: bool) -> List[Tuple[int, int]]:
    """Global ``[start, end)`` position ranges of the tokens a rank holds, in local order."""
    if not zig_zag:
        return [(rank * local_len, (rank + 1) * local_len)]
    c = local_len // 2
    return [(rank * c, (rank + 1) * c), ((2 * cp - 1 - rank) * c, (2 * cp - rank) * c)]


def _to_global_order(gathered: torch.Tensor, cp: int, zig_zag: bool) -> torch.Tensor:
    """``[cp, B, T_local, ...]`` (rank-major) -> ``[B, cp*T_local, ...]`` in global sequence order."""
    B, T_local = gathered.shape[1], gathered.shape[2]
    if not zig_zag:
        return gathered.transpose(0, 1).reshape(B, cp * T_local, *gathered.shape[3:])
    c = T_local // 2
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * cp)
    for r in range(cp):
        chunks[r] = gathered[r, :, :c]
        chunks[2 * cp - 1 - r] = gathered[r, :, c:]
    return torch.cat(chunks, dim=1)  # type: ignore[arg-type]


def ring_attention(backend, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, group, style,
                   cu_doc_lens: Optional[torch.Tensor] = None, cu_doc_lens_q: Optional[torch.Tensor] = None,
                   cu_doc_lens_k: Optional[torch.Tensor] = None, local_k_slice: Optional[slice] = None) -> torch.Tensor:
    """
    Causal attention of the local queries ``q [B, T_local, H, D]`` over the whole (sharded) sequence. ``backend`` is the
    attention backend whose ``_local`` computes attention on one device; ``style`` names the shard layout.
    """
    if cu_doc_lens is not None or cu_doc_lens_q is not None or cu_doc_lens_k is not None:
        raise NotImplementedError("document masking is not supported together with ring context parallelism yet")
    del local_k_slice
    from ..nn.attention.ring import RingAttentionLoadBalancerType

    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    zig_zag = style.load_balancer == RingAttentionLoadBalancerType.zig_zag
    T_local = q.shape[1]
    k_all = _to_global_order(_AllGatherSeq.apply(k, group), cp, zig_zag)
    v_all = _to_global_order(_AllGatherSeq.apply(v, group), cp, zig_zag)
    outs = []
    offset = 0
    for start, end in local_position_ranges(T_local, rank, cp, zig_zag):
        n = end - start
        q_chunk = q[:, offset: offset + n]
        # keys up to the chunk's last position; causal masking aligned at the end makes query i see keys <= start + i
        outs.append(backend._local(q_chunk, k_all[:, :end], v_all[:, :end], causal=True))
        offset += n
    return torch.cat(outs, dim=1) if len(outs) > 1 else outs[0]
