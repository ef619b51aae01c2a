"""
Context-parallel load balancers: how a sequence is split over CP ranks
(API of src/olmo_core/nn/attention/ring.py:13-549).

* zig-zag: the sequence is cut into ``2*CP`` chunks and rank ``r`` keeps chunks ``r`` and ``2CP-1-r`` so
  every rank gets the same amount of causal work;
* llama3: contiguous slices; keys/values are all-gathered, queries stay local (works with sliding
  windows and packed documents);
* ulysses: contiguous slices; attention runs head-parallel after an all-to-all.
"""

from __future__ import annotations

from abc import ABCMeta, abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.nn.functional as F

from ...config import Config, StrEnum
from ...distributed.utils import get_rank, get_world_size
from ...utils import ensure_multiple_of

__all__ = [
    "RingAttentionLoadBalancerType",
    "RingAttentionLoadBalancer",
    "RingAttentionZigZagLoadBalancer",
    "RingAttentionLlama3LoadBalancer",
    "UlyssesLoadBalancer",
    "RingContextParallelStyle",
    "UlyssesContextParallelStyle",
]


class RingAttentionLoadBalancerType(StrEnum):
    zig_zag = "zig_zag"
    llama3 = "llama3"
    ulysses = "ulysses"

    def build(self, cp_mesh) -> "RingAttentionLoadBalancer":
        pg = cp_mesh.get_group()
        kwargs = dict(cp_rank=get_rank(pg), cp_world_size=get_world_size(pg))
        if self == RingAttentionLoadBalancerType.zig_zag:
            return RingAttentionZigZagLoadBalancer(**kwargs)
        if self == RingAttentionLoadBalancerType.llama3:
            return RingAttentionLlama3LoadBalancer(**kwargs)
        return UlyssesLoadBalancer(**kwargs)


def _pad_dim(x: torch.Tensor, dim: int, amount: int, value: Union[int, float]) -> torch.Tensor:
    if amount <= 0:
        return x
    dim = dim % x.dim()
    pad = [0, 0] * (x.dim() - dim - 1) + [0, amount]
    return F.pad(x, pad, value=value)


class RingAttentionLoadBalancer(metaclass=ABCMeta):
    def __init__(self, *, cp_rank: int, cp_world_size: int):
        self.cp_rank = cp_rank
        self.cp_world_size = cp_world_size

    @abstractmethod
    def batch_shard(self, *, inputs: List[torch.Tensor], seq_dims: List[int],
                    pad_values: Optional[List[Union[int, float]]] = None,
                    length_multiple: Optional[int] = None) -> List[torch.Tensor]:
        raise NotImplementedError

    @abstractmethod
    def batch_shard_by_document(self, *, inputs: List[torch.Tensor], seq_dims: List[int], cu_doc_lens: torch.Tensor,
                                pad_values: Optional[List[Union[int, float]]] = None,
                                length_multiple: Optional[int] = None) -> Tuple[List[torch.Tensor], Dict[str, Any]]:
        raise NotImplementedError

    def pad(self, x: torch.Tensor, seq_dim: int, value: Union[int, float],
            length_multiple: Optional[int] = None) -> Tuple[torch.Tensor, int]:
        """``x`` padded at the end of ``seq_dim`` to a multiple of ``length_multiple`` (default: what this balancer's
        sharding needs), and the number of positions added."""
        multiple = length_multiple if length_multiple is not None else self._default_multiple()
        before = x.shape[seq_dim]
        out = self._padded(x, seq_dim, multiple, value)
        return out, out.shape[seq_dim] - before

    def _default_multiple(self) -> int:
        return self.cp_world_size

    def _padded(self, x: torch.Tensor, dim: int, multiple: int, value: Optional[Union[int, float]]) -> torch.Tensor:
        n = x.shape[dim]
        target = ensure_multiple_of(n, multiple)
        if target != n:
            if value is None:
                raise RuntimeError(f"sequence length {n} is not a multiple of {multiple} and no pad value was given")
            x = _pad_dim(x, dim, target - n, value)
        return x


class RingAttentionZigZagLoadBalancer(RingAttentionLoadBalancer):
    def _default_multiple(self) -> int:
        return 2 * self.cp_world_size

    def _take(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        chunks = x.chunk(2 * self.cp_world_size, dim=dim)
        return torch.cat((chunks[self.cp_rank], chunks[2 * self.cp_world_size - 1 - self.cp_rank]), dim=dim)

    def batch_shard(self, *, inputs, seq_dims, pad_values=None, length_multiple=None):
        if len(inputs) != len(seq_dims) or (pad_values is not None and len(pad_values) != len(inputs)):
            raise ValueError("'inputs', 'seq_dims' and 'pad_values' must have the same length")
        multiple = 2 * self.cp_world_size * (length_multiple or 1) if length_multiple else 2 * self.cp_world_size
        out = []
        for i, (x, dim) in enumerate(zip(inputs, seq_dims)):
            x = self._padded(x, dim, multiple, None if pad_values is None else pad_values[i])
            out.append(self._take(x, dim))
        return out

    def batch_shard_by_document(self, *, inputs, seq_dims, cu_doc_lens, pad_values=None, length_multiple=None):
        """Each document is split zig-zag on its own, so every rank holds ``1/CP`` of every document."""
        if cu_doc_lens.device.type != "cpu":
            raise RuntimeError("'cu_doc_lens' must live on the CPU for sharding")
        if cu_doc_lens[0] != 0:
            raise RuntimeError("'cu_doc_lens' must start with 0")
        multiple = 2 * self.cp_world_size * (length_multiple or 1)
        bounds = cu_doc_lens.tolist()
        out: List[torch.Tensor] = []
        new_lens: List[int] = []
        for i, (x, dim) in enumerate(zip(inputs, seq_dims)):
            if x.shape[0] != 1:
                raise RuntimeError("sharding by document needs batch size 1")
            pieces = []
            for d in range(len(bounds) - 1):
                doc = x.narrow(dim, bounds[d], bounds[d + 1] - bounds[d])
                doc = self._padded(doc, dim, multiple, None if pad_values is None else pad_values[i])
                if i == 0:
                    new_lens.append(doc.shape[dim] // self.cp_world_size)
                pieces.append(self._take(doc, dim))
            out.append(torch.cat(pieces, dim=dim))
        cu = torch.tensor([0] + new_lens, dtype=cu_doc_lens.dtype).cumsum(0).to(cu_doc_lens.dtype)
        return out, dict(cu_doc_lens=cu, max_doc_len=max(new_lens) if new_lens else 0)


class _ContiguousBalancer(RingAttentionLoadBalancer):
    def _slice(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        n = x.shape[dim] // self.cp_world_size
        return x.narrow(dim, self.cp_rank * n, n)

    def batch_shard(self, *, inputs, seq_dims, pad_values=None, length_multiple=None):
        multiple = self.cp_world_size * (length_multiple or 1)
        out = []
        for i, (x, dim) in enumerate(zip(inputs, seq_dims)):
            x = self._padded(x, dim, multiple, None if pad_values is None else pad_values[i])
            out.append(self._slice(x, dim))
        return out


class RingAttentionLlama3LoadBalancer(_ContiguousBalancer):
    def pad(self, x: torch.Tensor, seq_dim: int, padding_to_add: Union[int, float], value: Optional[Union[int, float]] = None,
            length_multiple: Optional[int] = None) -> Tuple[torch.Tensor, int]:
        """
        ``x`` with ``padding_to_add`` positions of ``value`` appended along ``seq_dim``
        (src/olmo_core/nn/attention/ring.py:380-388). Called as ``pad(x, seq_dim, value)`` or with ``length_multiple``
        it pads to a multiple instead, like the other balancers.
        """
        if value is None or length_multiple is not None:  # the generic form: (x, seq_dim, value, length_multiple)
            return super().pad(x, seq_dim, padding_to_add if value is None else value, length_multiple)
        return _pad_dim(x, seq_dim, int(padding_to_add), value), int(padding_to_add)

    def batch_shard_by_document(self, *, inputs, seq_dims, cu_doc_lens, pad_values=None, length_multiple=None):
        """
        Contiguous slice per rank plus what the varlen kernel needs: document boundaries as seen by the
        local queries (``cu_doc_lens_q``), by the keys those queries can reach (``cu_doc_lens_k``) and the
        slice of the gathered key sequence that covers them (``local_k_slice``).
        """
        if cu_doc_lens.device.type != "cpu":
            raise RuntimeError("'cu_doc_lens' must live on the CPU for sharding")
        shards = self.batch_shard(inputs=inputs, seq_dims=seq_dims, pad_values=pad_values, length_multiple=length_multiple)
        total = ensure_multiple_of(int(cu_doc_lens[-1]), self.cp_world_size * (length_multiple or 1))
        local = total // self.cp_world_size
        q_start, q_end = self.cp_rank * local, (self.cp_rank + 1) * local
        bounds = cu_doc_lens.tolist()
        if bounds[-1] < total:
            bounds.append(total)  # padding forms its own trailing document
        cu_q, cu_k = [0], [0]
        k_first: Optional[int] = None
        for d in range(len(bounds) - 1):
            s, e = bounds[d], bounds[d + 1]
            lo, hi = max(s, q_start), min(e, q_end)
            if lo >= hi:
                continue
            if k_first is None:
                k_first = s
            cu_q.append(cu_q[-1] + (hi - lo))
            cu_k.append(cu_k[-1] + (hi - s))  # keys from the document start up to the last local query
        k_first = k_first if k_first is not None else q_start
        extra = dict(
            cu_doc_lens_q=torch.tensor(cu_q, dtype=torch.int32),
            cu_doc_lens_k=torch.tensor(cu_k, dtype=torch.int32),
            max_doc_len_q=max((b - a) for a, b in zip(cu_q[:-1], cu_q[1:])) if len(cu_q) > 1 else 0,
            max_doc_len_k=max((b - a) for a, b in zip(cu_k[:-1], cu_k[1:])) if len(cu_k) > 1 else 0,
            local_k_slice=slice(k_first, q_end),
        )
        return shards, extra


class UlyssesLoadBalancer(_ContiguousBalancer):
    def batch_shard_by_document(self, *, inputs, seq_dims, cu_doc_lens, pad_values=None, length_multiple=None):
        """Attention sees the full sequence after the all-to-all, so document boundaries pass through unchanged."""
        shards = self.batch_shard(inputs=inputs, seq_dims=seq_dims, pad_values=pad_values, length_multiple=length_multiple)
        lens = (cu_doc_lens[1:] - cu_doc_lens[:-1]).tolist()
        return shards, dict(cu_doc_lens=cu_doc_lens, max_doc_len=max(lens) if lens else 0)


@dataclass
class RingContextParallelStyle(Config):
    """Ring attention: K/V blocks travel between ranks while queries stay put."""

    load_balancer: RingAttentionLoadBalancerType = RingAttentionLoadBalancerType.zig_zag
    head_stride: int = 1

    @classmethod
    def zig_zag(cls, head_stride: int = 1) -> "RingContextParallelStyle":
        return cls(load_balancer=RingAttentionLoadBalancerType.zig_zag, head_stride=head_stride)

    @classmethod
    def llama3(cls, head_stride: int = 1) -> "RingContextParallelStyle":
        return cls(load_balancer=RingAttentionLoadBalancerType.llama3, head_stride=head_stride)


@dataclass
class UlyssesContextParallelStyle(Config):
    """Ulysses: all-to-all from sequence-sharded to head-sharded tensors around a local attention."""

    @property
    def load_balancer(self) -> RingAttentionLoadBalancerType:
        return RingAttentionLoadBalancerType.ulysses
