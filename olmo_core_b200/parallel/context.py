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

On B200s with peer-mapped memory the gather disappears: :class:`KVExchange` keeps each rank's keys / values in a
symmetric buffer and the flash-attention kernels fetch every key / value tile from the GPU that owns it with TMA loads
over NVLink (``ops.attention.sharded_attention``), forward and backward; sliding windows skip the tiles (and the
NVLink traffic) they cannot see. Only the key / value gradients still travel through a reduce-scatter.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["ring_attention", "local_position_ranges", "KVExchange"]


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


class KVExchange:
    """
    Peer-mapped home of a context-parallel group's keys and values for the sharded attention kernels. Two modes:

    * ``push`` (default): ``publish`` launches one kernel per tensor that stores this rank's ``k, v [B, T_local, Hkv, D]``
      chunks straight into EVERY rank's sequence-ordered buffer ``[B, T, Hkv, D]`` over NVLink (ranks that cannot see a
      chunk -- later in the causal order, or beyond a sliding window -- are skipped, so a windowed layer only moves its
      halo). Every tile crosses NVLink once; after the barrier the attention kernels read local memory.
    * ``direct`` (``OLMO_CORE_B200_CP_KV=direct``): only a local copy is made and the attention kernels fetch every key /
      value tile from its owner with TMA loads over NVLink. No gathered copy exists, but a tile is re-read by every
      query tile that needs it (remote reads are not cached on the reading GPU), which costs more than it saves unless
      few query tiles share a key tile.

    Either way ``publish`` ends with a stream-ordered barrier and returns what the kernels need: the C arrays of K and V
    base addresses, the number of sources, the rows per batch entry in a source, and the tile layout. Two slots
    alternate, so one barrier per call is enough: a slot is rewritten only after a later barrier has shown that every
    peer's kernels that read it are done. One instance serves all layers of a model (the backward pass publishes a
    layer's K / V again instead of keeping ``n_layers`` peer-visible copies).
    """

    _instances: dict = {}

    def __init__(self, group, zig_zag: bool, mode: Optional[str] = None):
        import os

        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.zig_zag = zig_zag
        self.mode = mode or os.environ.get("OLMO_CORE_B200_CP_KV", "push")
        assert self.mode in ("push", "direct")
        self._buf = None
        self._numel = 0
        self._calls = 0
        self._arrays: dict = {}
        self._tables: dict = {}
        self._gbuf = None
        self._gnumel = 0
        self._gcalls = 0
        self._ghalf = None

    @classmethod
    def for_group(cls, group, zig_zag: bool) -> "KVExchange":
        import os

        key = (id(group), zig_zag, os.environ.get("OLMO_CORE_B200_CP_KV", "push"))
        if key not in cls._instances:
            cls._instances[key] = cls(group, zig_zag, key[2])
        return cls._instances[key]

    def _slot_arrays(self, slot: int, per_tensor: int, es: int):
        import ctypes

        if slot not in self._arrays:
            base = slot * 2 * per_tensor
            ptrs = [int(p) for p in self._buf.handle.buffer_ptrs]
            self._arrays[slot] = (
                (ctypes.c_void_p * self.world_size)(*[p + base * es for p in ptrs]),
                (ctypes.c_void_p * self.world_size)(*[p + (base + per_tensor) * es for p in ptrs]),
            )
        return self._arrays[slot]

    def _push_table(self, B: int, T_local: int, window: Optional[int], device):
        """Segments (source row, rows, destination rank, destination row) of this rank's chunks for every rank that sees them."""
        key = (B, T_local, window)
        if key not in self._tables:
            cp, T = self.world_size, T_local * self.world_size
            mine = local_position_ranges(T_local, self.rank, cp, self.zig_zag)
            rows = []
            piece = 1024  # rows per segment: the kernel gives every segment a fixed number of blocks
            for d in range(cp):
                theirs = local_position_ranges(T_local, d, cp, self.zig_zag)
                off = 0
                for a, b in mine:
                    # keys [a, b) are visible to queries [qa, qb) where they precede qb and, under a window, reach into
                    # [qa - (window - 1), ...): only that part (from its 128-row tile boundary on) is sent
                    lo, hi = b, a
                    for qa, qb in theirs:
                        first = max(a, ((qa - (window - 1)) // 128) * 128) if window else a
                        last = min(b, qb)
                        if first < last:
                            lo, hi = min(lo, first), max(hi, last)
                    for start in range(lo, hi, piece):
                        n = min(piece, hi - start)
                        rows += [(bi * T_local + off + start - a, n, d, bi * T + start) for bi in range(B)]
                    off += b - a
            cols = list(zip(*rows))
            self._tables[key] = (
                torch.tensor(cols[0], dtype=torch.int32, device=device), torch.tensor(cols[1], dtype=torch.int32, device=device),
                torch.tensor(cols[2], dtype=torch.int32, device=device), torch.tensor(cols[3], dtype=torch.int64, device=device),
            )
        return self._tables[key]

    def publish(self, k: torch.Tensor, v: torch.Tensor, layout, window: Optional[int] = None):
        import ctypes

        from ..ops import _lib
        from .symmetric import SymmetricBuffer

        n = k.numel()
        assert v.numel() == n and k.dtype == v.dtype and k.is_contiguous() and v.is_contiguous()
        per_tensor = n * self.world_size if self.mode == "push" else n
        if self._buf is None or per_tensor > self._numel or self._buf.tensor.dtype != k.dtype:
            self._buf = SymmetricBuffer(4 * per_tensor, k.dtype, k.device, self.group)  # [slot][K | V]
            self._numel = per_tensor
            self._arrays = {}
        slot = self._calls & 1
        self._calls += 1
        k_ptrs, v_ptrs = self._slot_arrays(slot, self._numel, k.element_size())
        B, T_local = k.shape[0], k.shape[1]
        if self.mode == "direct":
            base = slot * 2 * self._numel
            self._buf.tensor[base: base + n].view_as(k).copy_(k)
            self._buf.tensor[base + self._numel: base + self._numel + n].view_as(v).copy_(v)
            self._buf.barrier()
            return k_ptrs, v_ptrs, self.world_size, T_local, layout.c_array
        src_start, count, dst_rank, dst_start = self._push_table(B, T_local, window, k.device)
        cols = k.shape[2] * k.shape[3]
        status = _lib.status_buffer(k.device)
        for t, ptrs in ((k, k_ptrs), (v, v_ptrs)):
            rc = _lib.lib().ocb_moe_push_rows(
                t.data_ptr(), None, 1, src_start.data_ptr(), count.data_ptr(), dst_rank.data_ptr(), dst_start.data_ptr(),
                src_start.numel(), ctypes.cast(ptrs, ctypes.c_void_p), self.world_size, B * T_local * self.world_size, cols,
                cols, cols, status.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "ocb_moe_push_rows")
        self._buf.barrier()
        r = self.rank
        own_k = (ctypes.c_void_p * 1)(k_ptrs[r])
        own_v = (ctypes.c_void_p * 1)(v_ptrs[r])
        return own_k, own_v, 1, T_local * self.world_size, layout.gathered().c_array

    def grad_buffers(self, B: int, T: int, Hkv: int, D: int, dtype, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """
        Peer-visible ``[B, T, Hkv, D]`` homes (sequence order) for this rank's partial key / value gradients, from which
        ``reduce_to_owners`` lets every owner collect its rows. Two halves alternate like the K / V slots.
        """
        import os

        from .symmetric import SymmetricBuffer

        if os.environ.get("OLMO_CORE_B200_CP_GRAD", "peer") != "peer":
            return (torch.empty((B, T, Hkv, D), dtype=dtype, device=device),
                    torch.empty((B, T, Hkv, D), dtype=dtype, device=device))
        n = B * T * Hkv * D
        if self._gbuf is None or 2 * n > self._gnumel or self._gbuf.tensor.dtype != dtype:
            self._gbuf = SymmetricBuffer(4 * n, dtype, device, self.group)  # [half][dK | dV]
            self._gnumel = 2 * n
        half = self._gcalls & 1
        self._gcalls += 1
        base = half * self._gnumel
        self._ghalf = (half, n)
        flat = self._gbuf.tensor
        return flat[base: base + n].view(B, T, Hkv, D), flat[base + n: base + 2 * n].view(B, T, Hkv, D)

    def _reduce_table(self, B: int, T_local: int, window: Optional[int], device):
        """Segments of this rank's rows with the ranks whose queries can see them (both tensors: dK rows, then dV rows)."""
        key = ("reduce", B, T_local, window)
        if key not in self._tables:
            cp, T = self.world_size, T_local * self.world_size
            mine = local_position_ranges(T_local, self.rank, cp, self.zig_zag)
            piece, rows = 1024, []
            for which in range(2):  # dK, dV: the source holds [2, B * T] rows, the output [2, B * T_local]
                off = 0
                for a, b in mine:
                    for start in range(a, b, piece):
                        end = min(b, start + piece)
                        mask = 0
                        for p in range(cp):
                            for qa, qb in local_position_ranges(T_local, p, cp, self.zig_zag):
                                if start < qb and (not window or end > qa - (window - 1)):
                                    mask |= 1 << p
                        for bi in range(B):
                            rows.append((which * B * T + bi * T + start, which * B * T_local + bi * T_local + off + start - a,
                                         end - start, mask))
                    off += b - a
            cols = list(zip(*rows))
            self._tables[key] = (
                torch.tensor(cols[0], dtype=torch.int64, device=device), torch.tensor(cols[1], dtype=torch.int64, device=device),
                torch.tensor(cols[2], dtype=torch.int32, device=device), torch.tensor(cols[3], dtype=torch.int32, device=device),
            )
        return self._tables[key]

    def reduce_to_owners(self, dk_all: torch.Tensor, dv_all: torch.Tensor, window: Optional[int] = None
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[B, T, Hkv, D]`` partial gradients in global key order -> this rank's ``[B, T_local, Hkv, D]`` sums."""
        import ctypes

        from ..ops import _lib

        cp = self.world_size
        B, T = dk_all.shape[0], dk_all.shape[1]
        tail = tuple(dk_all.shape[2:])
        if self._gbuf is not None and self._ghalf is not None and dk_all.data_ptr() == (
                self._gbuf.tensor.data_ptr() + self._ghalf[0] * self._gnumel * dk_all.element_size()):
            # every owner sums its rows straight out of the peers' buffers (fp32, rank order): no packing, no collective
            half, n = self._ghalf
            self._ghalf = None
            self._gbuf.barrier()
            es = dk_all.element_size()
            ptrs = (ctypes.c_void_p * cp)(*[int(p) + half * self._gnumel * es for p in self._gbuf.handle.buffer_ptrs])
            src, dst, count, mask = self._reduce_table(B, T // cp, window, dk_all.device)
            out = torch.empty((2, B, T // cp) + tail, dtype=dk_all.dtype, device=dk_all.device)
            cols = tail[0] * tail[1]
            lib = _lib.lib()
            if not getattr(KVExchange, "_reduce_bound", False):
                from ctypes import c_int, c_longlong, c_void_p

                _lib.register_signature("ocb_peer_reduce_rows", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                                  c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p])
                KVExchange._reduce_bound = True
            rc = lib.ocb_peer_reduce_rows(ctypes.cast(ptrs, ctypes.c_void_p), cp, out.data_ptr(), src.data_ptr(),
                                          dst.data_ptr(), count.data_ptr(), mask.data_ptr(), src.numel(), cols, cols, cols,
                                          _lib.stream_ptr())
            _lib.check(rc, "ocb_peer_reduce_rows")
            return out[0], out[1]
        g = torch.stack([dk_all, dv_all])  # [2, B, T, ...]
        if self.zig_zag:
            order = [c for r in range(cp) for c in (r, 2 * cp - 1 - r)]
            g = g.view(2, B, 2 * cp, T // (2 * cp), *tail)[:, :, order]
        g = g.reshape(2, B, cp, T // cp, *tail).permute(2, 0, 1, 3, *range(4, 4 + len(tail))).contiguous()
        out = torch.empty_like(g[0])
        dist.reduce_scatter_tensor(out.view(-1), g.view(-1), op=dist.ReduceOp.SUM, group=self.group)
        return out[0], out[1]


def _sharded_kernels_usable(q: torch.Tensor, k: torch.Tensor, group, zig_zag: bool) -> bool:
    import os

    from ..ops.attention import has_flash_kernel
    from .symmetric import symmetric_memory_enabled

    if os.environ.get("OLMO_CORE_B200_CP_IN_KERNEL", "1") == "0":
        return False
    return (
        q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 128
        and q.shape[1] == k.shape[1] and q.shape[1] % (256 if zig_zag else 128) == 0
        and symmetric_memory_enabled(q.device, group) and has_flash_kernel()
    )


def ring_attention(backend, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, group, style,
                   cu_doc_lens: Optional[torch.Tensor] = None, cu_doc_lens_q: Optional[torch.Tensor] = None,
                   cu_doc_lens_k: Optional[torch.Tensor] = None, local_k_slice: Optional[slice] = None) -> torch.Tensor:
    """
    Causal attention of the local queries ``q [B, T_local, H, D]`` over the whole (sharded) sequence. ``backend`` is the
    attention backend whose ``_local`` computes attention on one device; ``style`` names the shard layout.
    """
    if cu_doc_lens_q is not None or cu_doc_lens_k is not None:
        raise NotImplementedError(
            "per-rank document lengths are not used here: the sequence is sharded by position and `cu_doc_lens` holds "
            "the document boundaries of the whole sequence")
    del local_k_slice
    from ..nn.attention.ring import RingAttentionLoadBalancerType

    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    zig_zag = style.load_balancer == RingAttentionLoadBalancerType.zig_zag
    T_local = q.shape[1]
    if _sharded_kernels_usable(q, k, group, zig_zag):
        from ..ops.attention import ShardedSequenceLayout, sharded_attention

        layout = ShardedSequenceLayout.for_rank(T_local, rank, cp, zig_zag)
        return sharded_attention(q, k.contiguous(), v.contiguous(), exchange=KVExchange.for_group(group, zig_zag),
                                 layout=layout, scale=getattr(backend, "scale", None),
                                 window_size=getattr(backend, "window", None), cu_seqlens=cu_doc_lens)
    k_all = _to_global_order(_AllGatherSeq.apply(k, group), cp, zig_zag)
    v_all = _to_global_order(_AllGatherSeq.apply(v, group), cp, zig_zag)
    outs = []
    offset = 0
    docs = None
    if cu_doc_lens is not None:
        # document of every position of the whole sequence, [B, T]: tokens attend inside their document only
        from ..ops.attention import _doc_ids

        docs = _doc_ids(cu_doc_lens.to(q.device), q.shape[0], cp * T_local)
    for start, end in local_position_ranges(T_local, rank, cp, zig_zag):
        n = end - start
        q_chunk = q[:, offset: offset + n]
        # keys up to the chunk's last position; causal masking aligned at the end makes query i see keys <= start + i
        if docs is None:
            outs.append(backend._local(q_chunk, k_all[:, :end], v_all[:, :end], causal=True))
        else:
            from ..ops.attention import _sdpa_path, attention_reference

            fn = _sdpa_path if q.is_cuda else attention_reference
            kw = dict(dropout_p=0.0) if q.is_cuda else {}
            outs.append(fn(q_chunk, k_all[:, :end], v_all[:, :end], causal=True, window_size=getattr(backend, "window", None),
                           cu_seqlens=None, cu_seqlens_k=None, scale=getattr(backend, "scale", None),
                           doc_ids=(docs[:, start:end], docs[:, :end]), **kw))
        offset += n
    return torch.cat(outs, dim=1) if len(outs) > 1 else outs[0]
