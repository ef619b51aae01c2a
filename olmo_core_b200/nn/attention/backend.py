"""
Attention backends (API of src/olmo_core/nn/attention/backend.py:43-1145).

There is one GPU implementation -- the in-tree flash-attention kernels reached through
``ops.attention.attention`` -- so the backend names the reference dispatches between third-party
packages (``flash_2``, ``flash_3``, ``flash_4``, ``te``) are accepted and all select
:class:`KernelAttentionBackend`. ``torch`` selects :class:`TorchAttentionBackend`, the masked-softmax /
SDPA statement of the same semantics that runs anywhere and serves as the oracle.

Context parallelism lives here too: Ulysses wraps the local attention in sequence<->head all-to-alls, the
ring styles gather keys/values across the CP group and attend with position-aware masks.
"""

from __future__ import annotations

import math
from abc import abstractmethod
from typing import Optional, Tuple, Type

import torch
import torch.distributed as dist
import torch.nn as nn

from ...config import StrEnum
from ...distributed.parallel.context_parallel import (
    all_to_all_cp2hp,
    all_to_all_single_cp2hp,
    all_to_all_single_hp2cp,
)
from ...exceptions import OLMoConfigurationError
from ...ops.attention import attention as attention_op
from ...ops.attention import attention_reference
from .kv_cache import KVCacheManager
from .ring import (
    RingAttentionLoadBalancerType,
    RingContextParallelStyle,
    UlyssesContextParallelStyle,
)

__all__ = [
    "AttentionBackendName",
    "AttentionBackend",
    "TorchAttentionBackend",
    "KernelAttentionBackend",
    "FlashAttention2Backend",
    "FlashAttention3Backend",
    "FlashAttention4Backend",
    "TEAttentionBackend",
]


class AttentionBackendName(StrEnum):
    torch = "torch"
    flash_2 = "flash_2"
    flash_3 = "flash_3"
    flash_4 = "flash_4"
    te = "te"

    def get_class(self) -> Type["AttentionBackend"]:
        return {
            AttentionBackendName.torch: TorchAttentionBackend,
            AttentionBackendName.flash_2: FlashAttention2Backend,
            AttentionBackendName.flash_3: FlashAttention3Backend,
            AttentionBackendName.flash_4: FlashAttention4Backend,
            AttentionBackendName.te: TEAttentionBackend,
        }[self]

    def build(self, **kwargs) -> "AttentionBackend":
        return self.get_class()(**kwargs)

    def assert_supported(self) -> None:
        self.get_class().assert_supported()

    def assert_supports_swa(self) -> None:
        self.get_class().assert_supports_swa()

    def assert_supports_ring_cp(self) -> None:
        self.get_class().assert_supports_ring_cp()

    def assert_supports_ulysses_cp(self) -> None:
        self.get_class().assert_supports_ulysses_cp()

    def assert_supports_packed_qkv(self) -> None:
        self.get_class().assert_supports_packed_qkv()

    def assert_supports_kv_cache(self) -> None:
        self.get_class().assert_supports_kv_cache()


class AttentionBackend(nn.Module):
    """
    Computes ``softmax(q k^T * scale + mask) v`` for ``q [B, Tq, H, D]``, ``k, v [B, Tk, Hkv, D]``.
    """

    def __init__(
        self,
        *,
        head_dim: int,
        n_heads: int,
        n_kv_heads: Optional[int] = None,
        scale: Optional[float] = None,
        dropout_p: float = 0.0,
        window_size: Tuple[int, int] = (-1, -1),
        cache: Optional[object] = None,
    ):
        super().__init__()
        self.head_dim = head_dim
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
        self.dropout_p = dropout_p
        self.window_size = window_size
        self.cp_pg: Optional[dist.ProcessGroup] = None
        self.cp_enabled = False
        self.ring: Optional[RingContextParallelStyle] = None
        self.uly: Optional[UlyssesContextParallelStyle] = None

    # -- capability checks ---------------------------------------------------------------------------
    @classmethod
    def assert_supported(cls) -> None:
        pass

    @classmethod
    def assert_supports_swa(cls) -> None:
        pass

    @classmethod
    def assert_supports_ring_cp(cls) -> None:
        pass

    @classmethod
    def assert_supports_ulysses_cp(cls) -> None:
        pass

    @classmethod
    def assert_supports_packed_qkv(cls) -> None:
        pass

    @classmethod
    def assert_supports_kv_cache(cls) -> None:
        pass

    @property
    def window(self) -> Optional[int]:
        """Number of keys a query may see (itself included), or None for full causal attention."""
        left = self.window_size[0]
        return None if left is None or left < 0 else left + 1

    def apply_cp(self, cp_mesh, ring: Optional[RingContextParallelStyle] = None,
                 uly: Optional[UlyssesContextParallelStyle] = None) -> None:
        if (ring is None) == (uly is None):
            raise OLMoConfigurationError("exactly one of 'ring' or 'uly' must be given")
        self.cp_pg = cp_mesh.get_group()
        self.cp_enabled = True
        self.ring, self.uly = ring, uly
        if ring is not None and ring.load_balancer == RingAttentionLoadBalancerType.zig_zag and self.window is not None:
            raise OLMoConfigurationError("zig-zag ring attention does not support sliding windows; use llama3 or ulysses")

    # -- the local computation ----------------------------------------------------------------------
    @abstractmethod
    def _local(self, q, k, v, *, cu_doc_lens=None, cu_doc_lens_k=None, max_doc_len=None, causal=True) -> torch.Tensor:
        raise NotImplementedError

    def warmup_cache(self, max_seq_len: int, device: torch.device) -> None:
        """
        Build whatever per-sequence-length buffers the backend caches (the reference's SDPA backend caches its
        sliding-window masks here). The kernels of this package derive their masks from per-row bounds computed on the
        fly, so there is nothing to prepare.
        """
        del max_seq_len, device

    def forward(
        self,
        qkv,
        cu_doc_lens: Optional[torch.Tensor] = None,
        cu_doc_lens_q: Optional[torch.Tensor] = None,
        cu_doc_lens_k: Optional[torch.Tensor] = None,
        max_doc_len: Optional[int] = None,
        max_doc_len_q: Optional[int] = None,
        max_doc_len_k: Optional[int] = None,
        local_k_slice: Optional[slice] = None,
        kv_cache: Optional[KVCacheManager] = None,
        cache_leftpad: Optional[torch.Tensor] = None,
        kv_cache_manager: Optional[KVCacheManager] = None,
    ) -> torch.Tensor:
        """``kv_cache_manager`` is the reference's name of ``kv_cache`` (src/olmo_core/nn/attention/backend.py:222-236)."""
        q, k, v = qkv
        kv_cache = kv_cache if kv_cache is not None else kv_cache_manager
        if kv_cache is not None:
            return self._decode(q, k, v, kv_cache, cache_leftpad)
        if not self.cp_enabled:
            return self._local(q, k, v, cu_doc_lens=cu_doc_lens, max_doc_len=max_doc_len)
        if self.uly is not None:
            q, k, v = all_to_all_cp2hp([q, k, v], self.cp_pg)
            out = self._local(q, k, v, cu_doc_lens=cu_doc_lens, max_doc_len=max_doc_len)
            return all_to_all_single_hp2cp(out, self.cp_pg)
        assert self.ring is not None
        from ...parallel.context import ring_attention

        return ring_attention(
            self, q, k, v, group=self.cp_pg, style=self.ring, cu_doc_lens_q=cu_doc_lens_q, cu_doc_lens_k=cu_doc_lens_k,
            local_k_slice=local_k_slice, cu_doc_lens=cu_doc_lens,
        )

    def _decode(self, q, k, v, kv_cache: KVCacheManager, cache_leftpad: Optional[torch.Tensor]) -> torch.Tensor:
        """Append to the cache and attend over everything cached (causal, aligned to the newest token)."""
        if cache_leftpad is not None:
            kv_cache.record_leftpad(cache_leftpad)
        kc, vc = kv_cache.append(k, v)
        B, Tq = q.shape[0], q.shape[1]
        Tk = kc.shape[1]
        leftpad = kv_cache.cache_leftpad
        pos_k = torch.arange(Tk, device=q.device)[None, :]
        pos_q = torch.arange(Tk - Tq, Tk, device=q.device)[None, :]
        mask = (pos_k[:, None, :] <= pos_q[:, :, None]) & (pos_k[:, None, :] >= leftpad[:, None, None])
        if self.window is not None:
            mask = mask & (pos_k[:, None, :] > pos_q[:, :, None] - self.window)
        qh = q.permute(0, 2, 1, 3)
        kh, vh = kc.permute(0, 2, 1, 3).to(q.dtype), vc.permute(0, 2, 1, 3).to(q.dtype)
        out = torch.nn.functional.scaled_dot_product_attention(
            qh, kh, vh, attn_mask=mask[:, None].expand(B, 1, Tq, Tk), scale=self.scale, enable_gqa=kh.shape[1] != qh.shape[1]
        )
        return torch.nan_to_num(out).permute(0, 2, 1, 3)


class TorchAttentionBackend(AttentionBackend):
    """Reference semantics with PyTorch ops only (CPU-capable)."""

    def _local(self, q, k, v, *, cu_doc_lens=None, cu_doc_lens_k=None, max_doc_len=None, causal=True):
        if q.is_cuda:
            from ...ops.attention import _sdpa_path

            return _sdpa_path(q, k, v, causal=causal, window_size=self.window, cu_seqlens=cu_doc_lens,
                              cu_seqlens_k=cu_doc_lens_k, scale=self.scale,
                              dropout_p=self.dropout_p if self.training else 0.0)
        return attention_reference(q, k, v, causal=causal, window_size=self.window, cu_seqlens=cu_doc_lens,
                                   cu_seqlens_k=cu_doc_lens_k, scale=self.scale,
                                   dropout_p=self.dropout_p if self.training else 0.0)


class KernelAttentionBackend(AttentionBackend):
    """The in-tree flash-attention kernels on CUDA; falls back to the reference math on CPU tensors."""

    def _local(self, q, k, v, *, cu_doc_lens=None, cu_doc_lens_k=None, max_doc_len=None, causal=True):
        if not q.is_cuda:
            return attention_reference(q, k, v, causal=causal, window_size=self.window, cu_seqlens=cu_doc_lens,
                                       cu_seqlens_k=cu_doc_lens_k, scale=self.scale)
        return attention_op(q, k, v, causal=causal, window_size=self.window, cu_seqlens=cu_doc_lens,
                            cu_seqlens_k=cu_doc_lens_k, max_seqlen=max_doc_len, scale=self.scale,
                            dropout_p=self.dropout_p if self.training else 0.0)


class FlashAttention2Backend(KernelAttentionBackend):
    pass


class FlashAttention3Backend(KernelAttentionBackend):
    pass


class FlashAttention4Backend(KernelAttentionBackend):
    pass


class TEAttentionBackend(KernelAttentionBackend):
    @classmethod
    def assert_supports_cp(cls) -> None:
        """Every context-parallel style is served by the in-tree kernels behind this backend name."""
