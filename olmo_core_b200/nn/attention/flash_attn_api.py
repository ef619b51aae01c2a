"""
Function-level attention entry points under the names that model code written against
src/olmo_core/nn/attention/flash_attn_api.py:37-518 expects. There is ONE attention implementation in this framework
(:func:`olmo_core_b200.ops.attention.attention`: the tcgen05 flash kernels on B200, masked softmax elsewhere), so every
``dispatch_*`` name routes to it; the ``has_*`` probes answer for that implementation rather than for external wheels.

Layouts follow the flash-attention convention: ``q [B, Tq, H, D]``, ``k, v [B, Tk, Hkv, D]``; with ``cu_seqlens`` the
batch holds packed documents and attention never crosses a document boundary.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ...ops.attention import attention, attention_reference, has_flash_kernel

__all__ = [
    "has_flash_attn_2", "has_flash_attn_3", "has_flash_attn_4", "has_ring_flash_attn",
    "dispatch_flash_attn", "dispatch_flash_attn_3", "dispatch_flash_attn_4",
    "dispatch_flash_attn_qkvpacked", "dispatch_flash_attn_3_qkvpacked",
    "dispatch_flash_attn_with_kvcache", "dispatch_flash_attn_3_with_kvcache",
    "dispatch_ring_flash_attn", "dispatch_ring_flash_attn_qkvpacked",
]


def has_flash_attn_2() -> bool:
    """True when the built-in flash kernels can run (a B200 with the kernel library loaded)."""
    return has_flash_kernel()


has_flash_attn_3 = has_flash_attn_2
has_flash_attn_4 = has_flash_attn_2


def has_ring_flash_attn() -> bool:
    """Context-parallel attention is built in and works on every backend (gloo included)."""
    return True


def _window(window_size: Tuple[Optional[int], Optional[int]], causal: bool) -> Optional[int]:
    """Flash-style ``(left, right)`` window → this framework's single window width (tokens to the left, inclusive)."""
    left, right = window_size
    if left is None or left < 0:
        return None
    if not causal and right not in (None, -1, 0):
        raise NotImplementedError("look-ahead windows are not supported")
    return int(left) + 1


def dispatch_flash_attn(q, k, v, *, cu_seqlens=None, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen=None,
                        max_seqlen_q=None, max_seqlen_k=None, dropout_p: float = 0.0,
                        softmax_scale: Optional[float] = None, causal: bool = False,
                        window_size: Tuple[int, int] = (-1, -1), **_unused) -> torch.Tensor:
    cu_q = cu_seqlens_q if cu_seqlens_q is not None else cu_seqlens
    cu_k = cu_seqlens_k if cu_seqlens_k is not None else cu_seqlens
    return attention(q, k, v, causal=causal, window_size=_window(window_size, causal), cu_seqlens=cu_q,
                     cu_seqlens_k=cu_k if cu_k is not cu_q else None,
                     max_seqlen=max_seqlen_q if max_seqlen_q is not None else max_seqlen, scale=softmax_scale,
                     dropout_p=dropout_p)


def dispatch_flash_attn_3(q, k, v, **kwargs) -> torch.Tensor:
    kwargs.pop("dropout_p", None)
    return dispatch_flash_attn(q, k, v, **kwargs)


def dispatch_flash_attn_4(q, k, v, *, seqused_k: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
    if seqused_k is not None:
        raise NotImplementedError("per-sequence key lengths are expressed with cu_seqlens_k here")
    return dispatch_flash_attn(q, k, v, **kwargs)


def dispatch_flash_attn_qkvpacked(qkv: torch.Tensor, *, cu_seqlens=None, max_seqlen=None, dropout_p: float = 0.0,
                                  softmax_scale: Optional[float] = None, causal: bool = False,
                                  window_size: Tuple[int, int] = (-1, -1)) -> torch.Tensor:
    """``qkv [B, T, 3, H, D]``: the three slices are strided views, no copy is made."""
    q, k, v = qkv.unbind(dim=2)
    return dispatch_flash_attn(q, k, v, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, dropout_p=dropout_p,
                               softmax_scale=softmax_scale, causal=causal, window_size=window_size)


def dispatch_flash_attn_3_qkvpacked(qkv: torch.Tensor, **kwargs) -> torch.Tensor:
    kwargs.pop("dropout_p", None)
    return dispatch_flash_attn_qkvpacked(qkv, **kwargs)


def dispatch_flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, cache_seqlens=None, cache_leftpad=None,
                                     softmax_scale: Optional[float] = None, causal: bool = False,
                                     window_size: Tuple[int, int] = (-1, -1)) -> torch.Tensor:
    """
    Decode-time attention over a ``[B, S_max, Hkv, D]`` cache. New ``k, v [B, T, Hkv, D]`` (if given) are first written
    at ``cache_seqlens`` (in place). Row ``b`` attends to cache slots ``[cache_leftpad[b], cache_seqlens[b] + T)``; with
    ``causal`` the last query lines up with the last valid key.
    """
    B, T = q.shape[:2]
    S = k_cache.shape[1]
    dev = q.device
    seqlens = (torch.zeros(B, dtype=torch.long, device=dev) if cache_seqlens is None
               else torch.as_tensor(cache_seqlens, device=dev).long().expand(B))
    t_new = 0
    if k is not None:
        assert v is not None
        t_new = k.shape[1]
        slots = seqlens[:, None] + torch.arange(t_new, device=dev)[None]  # [B, T]
        rows = torch.arange(B, device=dev)[:, None].expand_as(slots)
        k_cache[rows, slots] = k.to(k_cache.dtype)
        v_cache[rows, slots] = v.to(v_cache.dtype)
    end = seqlens + t_new  # first invalid slot, per row
    start = (torch.zeros_like(end) if cache_leftpad is None else torch.as_tensor(cache_leftpad, device=dev).long())
    key_pos = torch.arange(S, device=dev)[None, None, :]  # [1, 1, S]
    q_pos = (end[:, None] - T + torch.arange(T, device=dev)[None])[:, :, None]  # [B, T, 1] slot of each query
    mask = (key_pos >= start[:, None, None]) & (key_pos < end[:, None, None])
    if causal:
        mask = mask & (key_pos <= q_pos)
    width = _window(window_size, causal)
    if width is not None:
        mask = mask & (key_pos > q_pos - width)
    H, Hkv = q.shape[2], k_cache.shape[2]
    kk, vv = k_cache, v_cache
    if Hkv != H:
        kk, vv = kk.repeat_interleave(H // Hkv, dim=2), vv.repeat_interleave(H // Hkv, dim=2)
    out = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), kk.transpose(1, 2).to(q.dtype), vv.transpose(1, 2).to(q.dtype), attn_mask=mask[:, None].expand(B, 1, T, S),
        scale=softmax_scale)
    return out.transpose(1, 2)


dispatch_flash_attn_3_with_kvcache = dispatch_flash_attn_with_kvcache


def dispatch_ring_flash_attn(q, k, v, *, group: dist.ProcessGroup, strategy, cu_seqlens=None, cu_seqlens_q=None,
                             cu_seqlens_k=None, max_seqlen=None, max_seqlen_q=None, max_seqlen_k=None,
                             heads_k_stride: Optional[int] = None, local_k_slice: Optional[slice] = None,
                             dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False,
                             window_size: Tuple[int, int] = (-1, -1)) -> torch.Tensor:
    """Context-parallel attention: each rank holds a slice of the sequence laid out by ``strategy``."""
    from ...parallel.context import ring_attention
    from .backend import TorchAttentionBackend
    from .ring import RingAttentionLoadBalancerType, RingContextParallelStyle

    del heads_k_stride, local_k_slice, max_seqlen, max_seqlen_q, max_seqlen_k
    if dropout_p:
        raise NotImplementedError("dropout is not supported with context parallelism")
    if cu_seqlens_q is not None or cu_seqlens_k is not None:
        raise NotImplementedError("pass the document boundaries of the whole sequence as `cu_seqlens`")
    if not causal:
        raise NotImplementedError("context-parallel attention is causal")
    zig_zag = RingAttentionLoadBalancerType(strategy) == RingAttentionLoadBalancerType.zig_zag
    style = RingContextParallelStyle.zig_zag() if zig_zag else RingContextParallelStyle.llama3()
    backend = TorchAttentionBackend(head_dim=q.shape[-1], n_heads=q.shape[2], n_kv_heads=k.shape[2], scale=softmax_scale,
                                    window_size=window_size)
    return ring_attention(backend, q, k, v, group=group, style=style, cu_doc_lens=cu_seqlens)


def dispatch_ring_flash_attn_qkvpacked(qkv: torch.Tensor, *, group: dist.ProcessGroup, strategy, **kwargs) -> torch.Tensor:
    q, k, v = qkv.unbind(dim=2)
    kwargs.pop("cu_seqlens", None) if kwargs.get("cu_seqlens") is None else None
    return dispatch_ring_flash_attn(q, k, v, group=group, strategy=strategy, **kwargs)


def _reference(q, k, v, **kwargs):  # the oracle, exported for tests of code written against these entry points
    return attention_reference(q, k, v, **kwargs)
