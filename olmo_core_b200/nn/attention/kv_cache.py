"""
Key/value cache for incremental decoding (role of src/olmo_core/nn/attention/kv_cache.py:11-118).
Buffers are ``[B, S_max, H_kv, D]``; ``position`` is a host integer (the decode loop is host-driven, so
no device read-back is needed to know where to write).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

__all__ = ["KVCacheManager"]


class KVCacheManager(nn.Module):
    def __init__(self, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, device: torch.device,
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self._allocate(batch_size, max_seq_len, device, dtype)

    def _allocate(self, batch_size: int, max_seq_len: int, device, dtype) -> None:
        self._batch_size, self._max_seq_len = batch_size, max_seq_len
        shape = (batch_size, max_seq_len, self.num_kv_heads, self.head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, device=device, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape, device=device, dtype=dtype), persistent=False)
        self.register_buffer("cache_leftpad", torch.zeros(batch_size, dtype=torch.int32, device=device), persistent=False)
        self.position = 0

    def record_leftpad(self, leftpad: Optional[torch.Tensor]) -> None:
        if leftpad is not None:
            self.cache_leftpad.copy_(leftpad)

    def current_position(self) -> int:
        return self.position

    def append(self, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Write ``k, v [B, T, H_kv, D]`` at the current position; return views of everything cached so far."""
        t = k.shape[1]
        end = self.position + t
        if end > self._max_seq_len:
            raise RuntimeError(f"KV cache overflow: {end} > {self._max_seq_len}")
        self.k_cache[:, self.position:end].copy_(k)
        self.v_cache[:, self.position:end].copy_(v)
        self.position = end
        return self.k_cache[:, :end], self.v_cache[:, :end]

    def update_seqlen(self, seqlen: int) -> None:
        self.position += seqlen

    def zero_cache(self) -> None:
        self.k_cache.zero_()
        self.v_cache.zero_()
        self.cache_leftpad.zero_()
        self.position = 0

    def is_reusable(self, batch_size: int, max_seq_len: int) -> bool:
        return self._batch_size == batch_size and self._max_seq_len >= max_seq_len

    def reallocate(self, batch_size: int, max_seq_len: int, _explicitly_free_memory: bool = True) -> None:
        device, dtype = self.k_cache.device, self.k_cache.dtype
        del self.k_cache, self.v_cache, self.cache_leftpad
        if _explicitly_free_memory and device.type == "cuda":
            # the old cache can be most of the memory: hand it back before the new one is allocated
            import gc

            gc.collect()
            torch.cuda.empty_cache()
        self._allocate(batch_size, max_seq_len, device, dtype)

    def reset(self, batch_size: int, max_seq_len: int) -> None:
        if self.is_reusable(batch_size, max_seq_len):
            self.zero_cache()
        else:
            self.reallocate(batch_size, max_seq_len)
