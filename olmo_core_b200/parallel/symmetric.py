"""
Symmetric (peer-mapped) device memory for kernels that fuse compute with a collective.

A :class:`SymmetricBuffer` is a flat device tensor allocated identically on every rank of a process group and mapped
into every peer's address space over NVLink, so a kernel on one GPU can load from / store to the same offset of any
peer's buffer, and -- where the NVSwitch supports it -- through one multicast address that reaches all of them
(``multimem.ld_reduce`` / ``multimem.st``). Allocation and handle exchange use
``torch.distributed._symmetric_memory``; this module only adds what the kernels need: the peer pointers as a C
array, the multicast address, and a stream-ordered cross-rank barrier.

The barrier is this package's own kernel (``ops/csrc/peer_barrier_sm100.cu``): epoch flags in a small symmetric
buffer, published with ``st.release.sys`` and awaited with ``ld.acquire.sys`` under a deadline
(``OLMO_CORE_B200_BARRIER_TIMEOUT_MS``, default 60 s). A wait that runs out does not trap: the kernel records status
code 4 and returns, and :func:`olmo_core_b200.ops._lib.check_device_status` raises on the host, so a rank that died
between steps costs its peers one deadline instead of a hung GPU.

The fused optimizer step (:mod:`olmo_core_b200.ops.csrc.fused_optim_sm100`) keeps the gradient and low-precision
parameter buffers of the sharded-parameter runtime in such buffers. Set ``OLMO_CORE_B200_SYMMETRIC=0`` to fall back to
NCCL reduce-scatter / all-gather (also the automatic fallback when peer mapping is unavailable).
"""

from __future__ import annotations

import ctypes
import logging
import os
from typing import List, Optional

import torch
import torch.distributed as dist

log = logging.getLogger(__name__)

__all__ = ["SymmetricBuffer", "symmetric_memory_enabled", "ensure_symmetric_group"]

ENV_VAR = "OLMO_CORE_B200_SYMMETRIC"
MULTIMEM_ENV_VAR = "OLMO_CORE_B200_MULTIMEM"
BARRIER_TIMEOUT_ENV_VAR = "OLMO_CORE_B200_BARRIER_TIMEOUT_MS"


def symmetric_memory_enabled(device: torch.device, group: Optional[dist.ProcessGroup] = None) -> bool:
    """True when peer-mapped buffers should be used: CUDA device, NCCL group of more than one rank, not disabled."""
    if os.environ.get(ENV_VAR, "1") == "0" or device.type != "cuda":
        return False
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) < 2:
        return False
    if dist.get_world_size(group) > 16:  # the kernels take up to 16 peer pointers (one NVSwitch domain)
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True


def ensure_symmetric_group(group: Optional[dist.ProcessGroup]) -> str:
    """Make ``group`` known to the symmetric-memory allocator; returns its name."""
    group = group if group is not None else dist.group.WORLD
    return group.group_name  # groups are registered with the allocator lazily, at rendezvous


class SymmetricBuffer:
    """``numel`` elements of ``dtype`` at the same symmetric address on every rank of ``group``."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        ensure_symmetric_group(self.group)
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, self.group)
        self.world_size = self.handle.world_size
        self.rank = self.handle.rank
        ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        """C array of every rank's base address of this buffer, indexed by rank in the group."""
        mc = 0
        if os.environ.get(MULTIMEM_ENV_VAR, "1") != "0":
            try:
                if self.handle.has_multicast_support(device.type, device.index or 0):
                    mc = int(self.handle.multicast_ptr)
            except Exception:
                mc = 0
        self.multicast_ptr: Optional[int] = mc or None
        self._channel = 0
        # epoch flags of the barrier kernel: one row of 32-bit words per channel on every rank
        from ..ops import _lib

        words = _lib.lib().ocb_peer_barrier_flag_words()
        self._flags = symm.empty(words, dtype=torch.int32, device=device)
        self._flags.zero_()
        torch.cuda.synchronize(device)
        self._flag_handle = symm.rendezvous(self._flags, self.group)
        fptrs = [int(p) for p in self._flag_handle.buffer_ptrs]
        self._flag_ptrs = (ctypes.c_void_p * len(fptrs))(*fptrs)
        self._epochs = [0] * 8
        self.barrier_timeout_ms = int(os.environ.get(BARRIER_TIMEOUT_ENV_VAR, "60000"))
        dist.barrier(group=self.group)  # every rank's flags are zero before the first signal can arrive

    def barrier(self, channel: Optional[int] = None, *, timeout_ms: Optional[int] = None, _skip_signal_rank: int = -1) -> None:
        """
        Cross-rank barrier ordered with the current stream: work enqueued before it on every rank has finished, and its
        writes to peer memory are visible, before work enqueued after it starts. Bounded: see the module docstring.
        ``_skip_signal_rank`` (tests only) withholds this rank's signal from one peer so that the peer's wait runs out.
        """
        from ..ops import _lib

        ch = self._channel if channel is None else channel
        self._epochs[ch] += 1
        rc = _lib.lib().ocb_peer_barrier(self._flag_ptrs, self.world_size, self.rank, ch, self._epochs[ch] & 0xFFFFFFFF,
                                         self.barrier_timeout_ms if timeout_ms is None else timeout_ms, _skip_signal_rank,
                                         _lib.status_buffer(self.tensor.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ocb_peer_barrier")

    def __repr__(self) -> str:
        return (f"SymmetricBuffer(numel={self.tensor.numel()}, dtype={self.tensor.dtype}, world={self.world_size}, "
                f"multicast={'yes' if self.multicast_ptr else 'no'})")
