"""
Scaled-dot-product attention op: causal / sliding-window / packed-document (varlen) / GQA.

``attention`` takes ``q [B, Tq, H, D]`` and ``k, v [B, Tk, Hkv, D]`` (sequence-major, the layout the QKV
projection produces, so no transposes are needed on either side of the kernel). Semantics follow the
reference's attention backends (src/olmo_core/nn/attention/backend.py:299-444):

* causal masking aligned to the *end* of the key sequence (query ``i`` sees keys ``<= i + Tk - Tq``),
* ``window_size = w``: query ``i`` additionally only sees the last ``w`` keys ``[i-w+1, i]``,
* ``cu_seqlens``: documents packed along the (flattened) token dimension attend only within themselves.

On CUDA with bf16 inputs, ``head_dim`` 128, equal query / key lengths that are a multiple of 128, and neither a
sliding window nor document boundaries, the in-tree tcgen05 flash-attention kernels (``csrc/attention_sm100.cu``,
``csrc/attention_bwd_sm100.cu``) run forward and backward. Other cases take the masked PyTorch path.
``attention_reference`` is the plain fp32 restatement used on CPU and as the oracle in tests.
"""

from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from . import _lib

__all__ = ["attention", "attention_reference", "build_attention_mask", "has_flash_kernel", "sharded_attention",
           "ShardedSequenceLayout"]


def build_attention_mask(
    tq: int,
    tk: int,
    device: torch.device,
    *,
    causal: bool = True,
    window_size: Optional[int] = None,
    doc_ids_q: Optional[torch.Tensor] = None,
    doc_ids_k: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Boolean ``[tq, tk]`` (or ``[B, tq, tk]`` with document ids) mask, ``True`` = may attend."""
    qi = torch.arange(tq, device=device)[:, None] + (tk - tq)
    ki = torch.arange(tk, device=device)[None, :]
    mask = torch.ones(tq, tk, dtype=torch.bool, device=device)
    if causal:
        mask &= ki <= qi
    if window_size is not None and window_size > 0:
        mask &= ki > qi - window_size
    if doc_ids_q is not None and doc_ids_k is not None:
        mask = mask[None] & (doc_ids_q[:, :, None] == doc_ids_k[:, None, :])
    return mask


def _doc_ids(cu_seqlens: torch.Tensor, batch: int, t: int) -> torch.Tensor:
    flat = torch.arange(batch * t, device=cu_seqlens.device, dtype=cu_seqlens.dtype)
    return torch.bucketize(flat, cu_seqlens[1:], right=True).view(batch, t)


def attention_reference(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = True,
    window_size: Optional[int] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    dropout_p: float = 0.0,
    doc_ids: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
) -> torch.Tensor:
    """fp32 masked-softmax attention; returns ``[B, Tq, H, D]`` in ``q.dtype``. ``doc_ids`` gives the document of every
    query and of every key (``[B, Tq]``, ``[B, Tk]``) directly, for queries that are not the last ``Tq`` positions."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    if Hkv != H:
        rep = H // Hkv
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    dq = dk = None
    if doc_ids is not None:
        dq, dk = doc_ids
    elif cu_seqlens is not None:
        dq = _doc_ids(cu_seqlens, B, Tq)
        dk = _doc_ids(cu_seqlens_k if cu_seqlens_k is not None else cu_seqlens, B, Tk)
    mask = build_attention_mask(Tq, Tk, q.device, causal=causal, window_size=window_size, doc_ids_q=dq, doc_ids_k=dk)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask_b = mask[:, None] if mask.dim() == 3 else mask[None, None]
    scores = scores.masked_fill(~mask_b, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    probs = torch.nan_to_num(probs, nan=0.0)  # rows with no visible key
    if dropout_p > 0.0:
        probs = torch.nn.functional.dropout(probs, p=dropout_p)
    out = torch.matmul(probs, vf)
    return out.permute(0, 2, 1, 3).to(q.dtype)


_FLASH_BOUND = False


def has_flash_kernel() -> bool:
    """True when the loaded kernel library exports the attention entry points."""
    global _FLASH_BOUND
    if not _lib.available():
        return False
    lib = _lib.lib()
    if not hasattr(lib, "ocb_attention_fwd"):
        return False
    if not _FLASH_BOUND:
        _lib.register_signature(
            "ocb_attention_fwd",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_longlong, c_longlong, c_longlong, c_longlong, c_float, c_int, c_int, c_void_p, c_void_p],
        )
        _lib.register_signature(
            "ocb_attention_bwd",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_longlong, c_float, c_int,
             c_int, c_void_p, c_void_p],
        )
        if hasattr(lib, "ocb_attention_fwd_sharded"):
            _lib.register_signature(
                "ocb_attention_fwd_sharded",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                 c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_longlong, c_float, c_int, c_void_p, c_void_p],
            )
            _lib.register_signature(
                "ocb_attention_bwd_sharded",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
                 c_longlong, c_longlong, c_float, c_int, c_void_p, c_void_p],
            )
        _FLASH_BOUND = True
    return True


def _row_stride(t: torch.Tensor) -> int:
    # [B, T, H, D] tensors that are views into a wider row (e.g. a fused QKV buffer)
    return t.stride(1)


def _visibility_bounds(B: int, T: int, window: int, cu_seqlens: Optional[torch.Tensor], device, *, Tk: Optional[int] = None,
                       q_pos: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """
    int32 ``[B * Tq + B * Tk]`` for the flash kernels: per query the lowest visible key, then per key the position of the
    last query that sees it (key indices / query positions inside the ``Tk``-long sequence). One pair of arrays expresses
    sliding windows, document boundaries and both together; ``None`` when neither applies. Documents never span two rows
    of the batch (``cu_seqlens`` counts over ``B * Tk``). ``q_pos`` (int64 ``[Tq]``) gives the queries' positions when
    they are not the last ``Tq`` of the sequence (a shard of a context-parallel group).
    """
    if not window and cu_seqlens is None:
        return None
    Tk = T if Tk is None else Tk
    if q_pos is None:
        q_pos = torch.arange(Tk - T, Tk, device=device, dtype=torch.int64)
    tq = q_pos.to(device=device, dtype=torch.int64).repeat(B)
    tk = torch.arange(Tk, device=device, dtype=torch.int64).repeat(B)
    lo = torch.zeros_like(tq)
    hi = torch.full_like(tk, Tk - 1)
    if cu_seqlens is not None:
        # documents are ranges of the flattened [B * Tk] sequence; a query's document follows from its position
        cu = cu_seqlens.to(device=device, dtype=torch.int64)
        rows = torch.arange(B, device=device, dtype=torch.int64)
        base_q = rows.repeat_interleave(tq.numel() // B) * Tk
        base_k = rows.repeat_interleave(Tk) * Tk
        doc_q = torch.bucketize(base_q + tq, cu[1:], right=True).clamp(max=cu.numel() - 2)
        doc_k = torch.bucketize(base_k + tk, cu[1:], right=True).clamp(max=cu.numel() - 2)
        lo = torch.maximum(lo, cu[doc_q] - base_q)
        hi = torch.minimum(hi, cu[doc_k + 1] - 1 - base_k)
    if window:
        lo = torch.maximum(lo, tq - (window - 1))
        hi = torch.minimum(hi, tk + (window - 1))
    return torch.cat([lo, hi]).to(torch.int32).contiguous()


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, scale: float, causal: bool, window: int):  # type: ignore[override]
        B, Tq, H, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        q, k, v = (t if (t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == t.stride(1) * t.shape[1]) else t.contiguous()
                   for t in (q, k, v))
        out = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
        cu = _visibility_bounds(B, Tq, window, cu_seqlens, q.device, Tk=Tk)
        rc = _lib.lib().ocb_attention_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), _lib.ptr(cu),
            B, Tq, Tk, H, Hkv, D, _row_stride(q), _row_stride(k), _row_stride(v), _row_stride(out), scale,
            1 if causal else 0, window, _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_attention_fwd")
        ctx.save_for_backward(q, k, v, out, lse, cu if cu is not None else torch.empty(0, device=q.device))
        ctx.cfg = (scale, causal, window, cu is not None)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        q, k, v, out, lse, cu = ctx.saved_tensors
        scale, causal, window, has_cu = ctx.cfg
        B, Tq, H, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        dout = dout.contiguous()
        dq = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Tk, Hkv, D), dtype=k.dtype, device=k.device)
        dv = torch.empty((B, Tk, Hkv, D), dtype=v.dtype, device=v.device)
        delta = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
        rc = _lib.lib().ocb_attention_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr() if has_cu else None, delta.data_ptr(),
            B, Tq, Tk, H, Hkv, D, _row_stride(q), _row_stride(k), _row_stride(v), _row_stride(out), scale,
            1 if causal else 0, window, _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_attention_bwd")
        return dq, dk, dv, None, None, None, None


class ShardedSequenceLayout:
    """
    Where the tiles of a sequence that is sharded over a context-parallel group live, for the sharded attention kernels
    (``csrc/attn_seq_map.cuh``): the local queries are one or two chunks of ``q_chunk_tiles`` 128-row tiles that start
    at global tiles ``q_tile0``; the keys, in global order, are chunks of ``kv_chunk_tiles`` tiles, chunk ``c`` held by
    rank ``kv_chunks[c][0]`` from tile ``kv_chunks[c][1]`` of its local buffer.
    """

    def __init__(self, q_chunk_tiles: int, q_tile0: Tuple[int, int], kv_chunk_tiles: int, kv_chunks):
        self.q_chunk_tiles = int(q_chunk_tiles)
        self.q_tile0 = (int(q_tile0[0]), int(q_tile0[1]))
        self.kv_chunk_tiles = int(kv_chunk_tiles)
        self.kv_chunks = [(int(a), int(b)) for a, b in kv_chunks]
        flat = [self.q_chunk_tiles, *self.q_tile0, self.kv_chunk_tiles, len(self.kv_chunks)]
        for a, b in self.kv_chunks:
            flat += [a, b]
        self.c_array = (c_int * len(flat))(*flat)

    @classmethod
    def for_rank(cls, local_len: int, rank: int, cp: int, zig_zag: bool) -> "ShardedSequenceLayout":
        """Layout of rank ``rank`` holding ``local_len`` tokens: contiguous shards, or the mirrored zig-zag chunks."""
        if not zig_zag:
            tiles = local_len // 128
            return cls(tiles, (rank * tiles, 0), tiles, [(r, 0) for r in range(cp)])
        tiles = local_len // 256
        chunks = [(c, 0) if c < cp else (2 * cp - 1 - c, tiles) for c in range(2 * cp)]
        return cls(tiles, (rank * tiles, (2 * cp - 1 - rank) * tiles), tiles, chunks)

    def gathered(self) -> "ShardedSequenceLayout":
        """The same queries over keys that sit, in sequence order, in ONE buffer."""
        if getattr(self, "_gathered", None) is None:
            self._gathered = ShardedSequenceLayout(self.q_chunk_tiles, self.q_tile0, self.kv_chunk_tiles * len(self.kv_chunks),
                                                   [(0, 0)])
        return self._gathered

    def query_positions(self, device) -> torch.Tensor:
        """Global position of every local query row (int64)."""
        n = self.q_chunk_tiles * 128
        parts = [torch.arange(self.q_tile0[0] * 128, self.q_tile0[0] * 128 + n, device=device)]
        if self.q_tile0[1]:
            parts.append(torch.arange(self.q_tile0[1] * 128, self.q_tile0[1] * 128 + n, device=device))
        return torch.cat(parts)


class _ShardedFlashAttention(torch.autograd.Function):
    """Attention of local queries over keys / values that stay on their owners (see :func:`sharded_attention`)."""

    @staticmethod
    def forward(ctx, q, k, v, exchange, layout, scale: float, window: int, cu_seqlens=None):  # type: ignore[override]
        B, Tq, H, D = q.shape
        T_local, Hkv = k.shape[1], k.shape[2]
        Tk = layout.kv_chunk_tiles * 128 * len(layout.kv_chunks)
        q = q.contiguous()
        k_ptrs, v_ptrs, n_src, rows_src, kv_layout = exchange.publish(k, v, layout, window or None)
        out = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
        bounds = _visibility_bounds(B, Tq, window, cu_seqlens, q.device, Tk=Tk, q_pos=layout.query_positions(q.device)[:Tq])
        ld_kv = Hkv * D
        rc = _lib.lib().ocb_attention_fwd_sharded(
            q.data_ptr(), k_ptrs, v_ptrs, n_src, rows_src, kv_layout, out.data_ptr(), lse.data_ptr(),
            _lib.ptr(bounds), B, Tq, Tk, H, Hkv, D, _row_stride(q), ld_kv, ld_kv, _row_stride(out), scale, 1,
            _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_attention_fwd_sharded")
        ctx.save_for_backward(q, k, v, out, lse, bounds if bounds is not None else torch.empty(0, device=q.device))
        ctx.cfg = (exchange, layout, scale, bounds is not None, Tk, window)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        q, k, v, out, lse, bounds = ctx.saved_tensors
        exchange, layout, scale, has_bounds, Tk, window = ctx.cfg
        B, Tq, H, D = q.shape
        T_local, Hkv = k.shape[1], k.shape[2]
        dout = dout.contiguous()
        # the peers' K / V of this layer are needed once more
        k_ptrs, v_ptrs, n_src, rows_src, kv_layout = exchange.publish(k, v, layout, window or None)
        dq = torch.empty((B, Tq, H, D), dtype=q.dtype, device=q.device)
        if hasattr(exchange, "grad_buffers"):
            dk_all, dv_all = exchange.grad_buffers(B, Tk, Hkv, D, k.dtype, k.device)
        else:
            dk_all = torch.empty((B, Tk, Hkv, D), dtype=k.dtype, device=k.device)
            dv_all = torch.empty((B, Tk, Hkv, D), dtype=v.dtype, device=v.device)
        delta = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device)
        ld_kv = Hkv * D
        rc = _lib.lib().ocb_attention_bwd_sharded(
            q.data_ptr(), k_ptrs, v_ptrs, n_src, rows_src, kv_layout, out.data_ptr(), dout.data_ptr(),
            lse.data_ptr(), dq.data_ptr(), dk_all.data_ptr(), dv_all.data_ptr(), bounds.data_ptr() if has_bounds else None,
            delta.data_ptr(), B, Tq, Tk, H, Hkv, D, _row_stride(q), ld_kv, ld_kv, _row_stride(out), scale, 1,
            _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr(),
        )
        _lib.check(rc, "ocb_attention_bwd_sharded")
        dk, dv = exchange.reduce_to_owners(dk_all, dv_all, window or None)
        return dq, dk, dv, None, None, None, None, None


def sharded_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, exchange, layout: ShardedSequenceLayout,
                      scale: Optional[float] = None, window_size: Optional[int] = None,
                      cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """
    Causal attention of this rank's queries ``q [B, T_local, H, 128]`` over the whole sequence of a context-parallel
    group. ``k, v [B, T_local, Hkv, 128]`` are this rank's keys / values. ``exchange``
    (:class:`olmo_core_b200.parallel.context.KVExchange`) moves them through peer-mapped memory -- pushed once into every
    rank's sequence-ordered buffer, or left with their owner and read tile by tile by the kernels -- and tells the
    kernels where each key / value tile is. Sliding windows are supported; key / value gradients are summed onto
    their owners by ``exchange.reduce_to_owners``. ``cu_seqlens`` are the cumulative document lengths of the WHOLE
    (unsharded, flattened ``[B * T]``) sequence: tokens only attend inside their document, wherever its pieces live.
    """
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _ShardedFlashAttention.apply(q, k, v, exchange, layout, scale, int(window_size or 0), cu_seqlens)


def _sdpa_path(q, k, v, *, causal, window_size, cu_seqlens, cu_seqlens_k, scale, dropout_p, doc_ids=None):
    """Masked ``scaled_dot_product_attention``: used for dtypes / head sizes the flash kernel does not take."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    mask = None
    is_causal = causal and Tq == Tk and window_size is None and cu_seqlens is None and doc_ids is None
    if not is_causal and (causal or window_size is not None or cu_seqlens is not None or doc_ids is not None):
        dq = dk = None
        if doc_ids is not None:
            dq, dk = doc_ids
        elif cu_seqlens is not None:
            dq = _doc_ids(cu_seqlens, B, Tq)
            dk = _doc_ids(cu_seqlens_k if cu_seqlens_k is not None else cu_seqlens, B, Tk)
        mask = build_attention_mask(Tq, Tk, q.device, causal=causal, window_size=window_size, doc_ids_q=dq, doc_ids_k=dk)
        mask = mask[:, None] if mask.dim() == 3 else mask
    out = torch.nn.functional.scaled_dot_product_attention(
        qh, kh, vh, attn_mask=mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale, enable_gqa=Hkv != H
    )
    return out.permute(0, 2, 1, 3)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = True,
    window_size: Optional[int] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    scale: Optional[float] = None,
    dropout_p: float = 0.0,
) -> torch.Tensor:
    """See the module docstring. Returns ``[B, Tq, H, D]``."""
    D = q.shape[-1]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    use_flash = (
        q.is_cuda
        and q.dtype == torch.bfloat16
        and k.dtype == torch.bfloat16
        and v.dtype == torch.bfloat16
        and D == 128
        and dropout_p == 0.0
        and cu_seqlens_k is None
        and (causal or (cu_seqlens is None and not window_size))
        and (q.shape[1] == k.shape[1] or (causal and cu_seqlens is None and q.shape[1] < k.shape[1]))
        and q.shape[1] % 128 == 0
        and k.shape[1] % 128 == 0
        and has_flash_kernel()
    )
    if use_flash:
        return _FlashAttention.apply(q, k, v, cu_seqlens, scale, bool(causal), int(window_size or 0))
    return _sdpa_path(q, k, v, causal=causal, window_size=window_size, cu_seqlens=cu_seqlens,
                      cu_seqlens_k=cu_seqlens_k, scale=scale, dropout_p=dropout_p)
