"""
Ulysses sequence <-> head exchange over peer memory
(role of ``all_to_all_single_cp2hp`` / ``all_to_all_single_hp2cp`` in
src/olmo_core/distributed/parallel/context_parallel.py:60-200, where each is permute + contiguous copy, an NCCL
all-to-all, and a second permute + copy).

Here one kernel (``ocb_push_row_slices``) does the transpose and the transfer: for ``cp2hp`` every rank stores head group
``d`` of each of its tokens straight into rank ``d``'s ``[B, T, H/CP, D]`` receive buffer at the token's global position;
``hp2cp`` stores the tokens of sequence shard ``d`` into rank ``d``'s ``[B, T/CP, H, D]`` buffer at this rank's head
columns. No packing copy exists on the sending side and the data lands in its final layout; a stream-ordered barrier
across the ranks completes the exchange. The receive buffers are symmetric memory, double-buffered (a half is
overwritten only after a later barrier has shown that its readers are done), and the result is copied out of them once
because autograd may keep it for the backward pass. Each direction is the other's gradient.

``OLMO_CORE_B200_ULYSSES_PEER=0`` (or tensors the kernel does not take) falls back to the all-to-all path.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib

__all__ = ["peer_exchange_usable", "cp2hp", "hp2cp"]

_SIG = False
_PIECE = 1024  # rows per segment: the kernel gives every segment a fixed number of blocks


def _bind() -> bool:
    global _SIG
    if not _lib.available() or not hasattr(_lib.lib(), "ocb_push_row_slices"):
        return False
    if not _SIG:
        from ctypes import c_int, c_longlong, c_void_p

        _lib.register_signature(
            "ocb_push_row_slices",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong,
             c_int, c_longlong, c_longlong, c_void_p, c_void_p])
        _SIG = True
    return True


def peer_exchange_usable(x: torch.Tensor, group) -> bool:
    from .symmetric import symmetric_memory_enabled

    if os.environ.get("OLMO_CORE_B200_ULYSSES_PEER", "1") == "0":
        return False
    return (x.is_cuda and x.dim() == 4 and x.element_size() == 2 and x.shape[3] % 8 == 0
            and symmetric_memory_enabled(x.device, group) and _bind())


class _Exchange:
    """Receive buffers and segment tables of one process group."""

    _instances: Dict[int, "_Exchange"] = {}

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._buf = None
        self._numel = 0
        self._turn = 0
        self._tables: dict = {}

    @classmethod
    def of(cls, group) -> "_Exchange":
        if id(group) not in cls._instances:
            cls._instances[id(group)] = cls(group)
        return cls._instances[id(group)]

    def _half(self, numel: int, dtype, device):
        from .symmetric import SymmetricBuffer

        if self._buf is None or numel > self._numel or self._buf.tensor.dtype != dtype:
            self._buf = SymmetricBuffer(2 * numel, dtype, device, self.group)
            self._numel = numel
        turn = self._turn
        self._turn ^= 1
        es = self._buf.tensor.element_size()
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) + turn * self._numel * es for p in self._buf.handle.buffer_ptrs])
        return self._buf.tensor[turn * self._numel: turn * self._numel + numel], ptrs

    def _table(self, to_heads: bool, B: int, t: int, h: int, D: int, device) -> Tuple[torch.Tensor, ...]:
        """Segments of one direction; ``t`` tokens per shard, ``h`` heads per group."""
        key = (to_heads, B, t, h, D)
        if key not in self._tables:
            cp, r = self.world, self.rank
            seg = []
            for d in range(cp):
                for b in range(B):
                    for s in range(0, t, _PIECE):
                        n = min(_PIECE, t - s)
                        if to_heads:  # my tokens' head group d -> rank d, rows of my sequence shard
                            seg.append((b * t + s, n, d, b * cp * t + r * t + s, d * h * D // 8, 0))
                        else:         # sequence shard d of my head group -> rank d, my head columns
                            seg.append((b * cp * t + d * t + s, n, d, b * t + s, 0, r * h * D // 8))
            cols = list(zip(*seg))
            i32 = dict(dtype=torch.int32, device=device)
            self._tables[key] = (torch.tensor(cols[0], **i32), torch.tensor(cols[1], **i32), torch.tensor(cols[2], **i32),
                                 torch.tensor(cols[3], dtype=torch.int64, device=device), torch.tensor(cols[4], **i32),
                                 torch.tensor(cols[5], **i32))
        return self._tables[key]

    def run(self, x: torch.Tensor, to_heads: bool) -> torch.Tensor:
        cp = self.world
        x = x.contiguous()
        if to_heads:
            B, t, H, D = x.shape
            h = H // cp
            out_shape, ld_src, ld_dst, dst_rows = (B, cp * t, h, D), H * D, h * D, B * cp * t
        else:
            B, T, h, D = x.shape
            t = T // cp
            out_shape, ld_src, ld_dst, dst_rows = (B, t, cp * h, D), h * D, cp * h * D, B * t
        recv, ptrs = self._half(x.numel(), x.dtype, x.device)
        tab = self._table(to_heads, B, t, h, D, x.device)
        rc = _lib.lib().ocb_push_row_slices(
            x.data_ptr(), tab[0].data_ptr(), tab[1].data_ptr(), tab[2].data_ptr(), tab[3].data_ptr(), tab[4].data_ptr(),
            tab[5].data_ptr(), tab[0].numel(), ctypes.cast(ptrs, ctypes.c_void_p), cp, dst_rows, h * D, ld_src, ld_dst,
            _lib.status_buffer(x.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_push_row_slices")
        self._buf.barrier()
        return recv.view(out_shape).clone()


class _PeerExchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, to_heads: bool):  # type: ignore[override]
        ctx.group, ctx.to_heads = group, to_heads
        return _Exchange.of(group).run(x, to_heads)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _Exchange.of(ctx.group).run(g, not ctx.to_heads), None, None


def cp2hp(x: torch.Tensor, group: Optional[dist.ProcessGroup]) -> torch.Tensor:
    """``[B, T/CP, H, D] -> [B, T, H/CP, D]`` (autograd-aware)."""
    return _PeerExchange.apply(x, group if group is not None else dist.group.WORLD, True)


def hp2cp(x: torch.Tensor, group: Optional[dist.ProcessGroup]) -> torch.Tensor:
    """``[B, T, H/CP, D] -> [B, T/CP, H, D]`` (autograd-aware)."""
    return _PeerExchange.apply(x, group if group is not None else dist.group.WORLD, False)
