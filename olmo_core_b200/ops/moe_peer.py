"""
Expert-parallel token exchange over NVLink peer memory.

The dropless expert-parallel layer of the reference (src/olmo_core/nn/moe/parallel_mlp.py, ``parallel_forward_once``)
gathers tokens into a send buffer, runs an NCCL all-to-all, re-sorts what it received by local expert, and mirrors all of
that on the way back, with host synchronisations to size the variable splits. Here the permutation and the transfer are ONE
kernel (``ocb_moe_push_rows``): every rank stores each of its expert-sorted rows straight into the receive buffer of the GPU
that owns the row's expert, at an offset computed on the device from the all-gathered routing counts, so that the rows land
already grouped by local expert. The way back uses the same kernel with the transposed segment table.

Buffers are symmetric (same address on every rank, peer-mapped) and double-buffered: a transfer is "launch the push kernel,
then a stream-ordered cross-rank barrier", and because every rank issues the same sequence of transfers, the barrier of
transfer ``k+1`` also proves that everybody has finished reading the buffer half that transfer ``k+2`` overwrites.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .moe import _inverse, _scatter_rows

__all__ = ["PeerExpertExchange", "peer_exchange_enabled", "SegmentTables"]

ENV_VAR = "OLMO_CORE_B200_EP_PEER"


def peer_exchange_enabled(x: torch.Tensor, group: Optional[dist.ProcessGroup]) -> bool:
    from ..parallel.symmetric import symmetric_memory_enabled

    return (
        os.environ.get(ENV_VAR, "1") != "0"
        and x.is_cuda
        and x.dtype == torch.bfloat16
        and x.dim() == 2
        and x.shape[1] % 8 == 0
        and x.stride(1) == 1
        and symmetric_memory_enabled(x.device, group)
    )


@dataclass
class SegmentTables:
    """Device-side description of one routing decision, shared by the four transfers of a layer's forward and backward."""

    to_experts: Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]  # src_start, count, dst_rank, dst_start
    to_tokens: Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]
    offsets: torch.Tensor  # int32 [E_local + 1]: row ranges of the local experts in the receive layout
    total: torch.Tensor    # int32 scalar: rows this rank receives


class _Half:
    """One of the two halves of a double-buffered symmetric buffer: a local view plus every peer's address of it."""

    def __init__(self, buf, offset_elems: int, rows: int, cols: int):
        self.view = buf.tensor[offset_elems: offset_elems + rows * cols].view(rows, cols)
        ptrs = [int(p) + offset_elems * buf.tensor.element_size() for p in buf.handle.buffer_ptrs]
        self.peer_ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)


class PeerExpertExchange:
    """Symmetric receive (expert side) and return (token side) buffers of one expert-parallel group and row width."""

    _cache: Dict[Tuple[int, int, int], "PeerExpertExchange"] = {}

    @classmethod
    def get(cls, group: dist.ProcessGroup, cols: int, rows: int, device: torch.device) -> "PeerExpertExchange":
        key = (id(group), cols, device.index or 0)
        ex = cls._cache.get(key)
        if ex is None or ex.rows < rows:
            ex = cls(group, cols, rows, device)
            cls._cache[key] = ex
        return ex

    def __init__(self, group: dist.ProcessGroup, cols: int, rows: int, device: torch.device,
                 capacity_factor: Optional[float] = None):
        from ..parallel.symmetric import SymmetricBuffer

        self.group, self.cols, self.rows = group, cols, rows
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        factor = capacity_factor or float(os.environ.get("OLMO_CORE_B200_EP_CAPACITY", "2.0"))
        # a perfectly balanced router sends every rank `rows` rows; `factor` is the head-room for imbalance
        self.capacity = min(int(rows * factor) + 128, rows * self.world)
        self._recv = SymmetricBuffer(2 * self.capacity * cols, torch.bfloat16, device, group)
        self._ret = SymmetricBuffer(2 * rows * cols, torch.bfloat16, device, group)
        self._recv_halves = [_Half(self._recv, h * self.capacity * cols, self.capacity, cols) for h in range(2)]
        self._ret_halves = [_Half(self._ret, h * rows * cols, rows, cols) for h in range(2)]
        self._recv_turn = self._ret_turn = 0
        self.transfers = 0

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def tables(self, counts: torch.Tensor, num_local_experts: int) -> SegmentTables:
        """``counts``: rows this rank routes to every global expert, ``[E]``. Communicates ``E`` integers per rank."""
        ep, me, e_local = self.world, self.rank, num_local_experts
        E = ep * e_local
        counts = counts.to(torch.int32).contiguous()
        counts_all = torch.empty((ep, E), dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(counts_all.view(-1), counts, group=self.group)
        # receive layout of rank p: rows grouped by (local expert, source rank), row-major
        flat = counts_all.t().contiguous().view(ep, e_local * ep).to(torch.int64)
        base = flat.cumsum(1) - flat
        sorted_start = counts_all.to(torch.int64).cumsum(1) - counts_all  # [source rank, expert]: start in its sorted rows
        arange_e = torch.arange(E, device=counts.device, dtype=torch.int32)
        to_experts = (
            sorted_start[me].to(torch.int32).contiguous(),
            counts,
            (arange_e // e_local).contiguous(),
            base.view(E, ep)[:, me].contiguous(),
        )
        to_tokens = (
            base[me].to(torch.int32).contiguous(),
            flat[me].to(torch.int32).contiguous(),
            torch.arange(ep, device=counts.device, dtype=torch.int32).repeat(e_local).contiguous(),
            sorted_start[:, me * e_local:(me + 1) * e_local].t().reshape(-1).contiguous(),
        )
        per_expert = flat[me].view(e_local, ep).sum(1)
        offsets = torch.zeros(e_local + 1, dtype=torch.int32, device=counts.device)
        offsets[1:] = per_expert.cumsum(0).to(torch.int32)
        return SegmentTables(to_experts, to_tokens, offsets, offsets[-1])

    def _push(self, src: torch.Tensor, gather_idx: Optional[torch.Tensor], gather_div: int, table, half: _Half,
              capacity: int) -> None:
        src_start, count, dst_rank, dst_start = table
        status = _lib.status_buffer(src.device)
        rc = _lib.lib().ocb_moe_push_rows(
            src.data_ptr(), _lib.ptr(gather_idx), gather_div, src_start.data_ptr(), count.data_ptr(), dst_rank.data_ptr(),
            dst_start.data_ptr(), src_start.numel(), ctypes.cast(half.peer_ptrs, ctypes.c_void_p), self.world, capacity,
            self.cols, src.stride(0), self.cols, status.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_moe_push_rows")
        self.transfers += 1

    def to_experts(self, src: torch.Tensor, gather_idx: Optional[torch.Tensor], gather_div: int, t: SegmentTables) -> torch.Tensor:
        """Deliver expert-sorted rows to the owners of their experts; returns this rank's receive buffer ``[capacity, cols]``
        whose first ``t.offsets[-1]`` rows (a device-side count) are the received rows, grouped by local expert."""
        half = self._recv_halves[self._recv_turn]
        self._recv_turn ^= 1
        self._push(src, gather_idx, gather_div, t.to_experts, half, self.capacity)
        self._recv.barrier()
        # No host read: the whole receive half is handed on (rows past the last group belong to no expert: the grouped
        # kernels never read them as data), and a rank that is sent more rows than the half holds is caught on the device
        # (the push kernel skips them and sets the status word; `check_device_status` raises, naming the capacity knob).
        return half.view.clone()

    def to_tokens(self, src: torch.Tensor, t: SegmentTables, n_rows: int, clone: bool) -> torch.Tensor:
        """Return rows in the receive layout to the ranks (and sorted positions) they came from; ``[n_rows, cols]``."""
        half = self._ret_halves[self._ret_turn]
        self._ret_turn ^= 1
        self._push(src, None, 1, t.to_tokens, half, self.rows)
        self._ret.barrier()
        out = half.view[:n_rows]
        return out.clone() if clone else out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, indices, top_k: int, ex: PeerExpertExchange, t: SegmentTables):  # type: ignore[override]
        ctx.ex, ctx.t, ctx.top_k, ctx.n_rows = ex, t, top_k, indices.numel()
        ctx.save_for_backward(_inverse(indices))
        return ex.to_experts(x, indices, top_k, t)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        (inverse,) = ctx.saved_tensors
        back = ctx.ex.to_tokens(grad.contiguous(), ctx.t, ctx.n_rows, clone=False)
        return _scatter_rows(back, inverse, None, ctx.top_k), None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, n_rows: int, ex: PeerExpertExchange, t: SegmentTables):  # type: ignore[override]
        ctx.ex, ctx.t = ex, t
        return ex.to_tokens(ys.contiguous(), t, n_rows, clone=True)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        return ctx.ex.to_experts(grad.contiguous(), None, 1, ctx.t), None, None, None


def dispatch(x: torch.Tensor, indices: torch.Tensor, top_k: int, ex: PeerExpertExchange, t: SegmentTables) -> torch.Tensor:
    """``x``: ``[N, d]`` tokens; ``indices``: the expert sort of the ``N * top_k`` routed copies. Returns the rows this
    rank's experts process, grouped by local expert (``t.offsets``)."""
    return _Dispatch.apply(x, indices, top_k, ex, t)


def combine(ys: torch.Tensor, n_rows: int, ex: PeerExpertExchange, t: SegmentTables) -> torch.Tensor:
    """Inverse of :func:`dispatch` for the expert outputs: ``[n_rows, d]`` in the sender's expert-sorted order."""
    return _Combine.apply(ys, n_rows, ex, t)
