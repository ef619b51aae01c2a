"""
Context-parallel configuration and the Ulysses sequence<->head exchanges
(src/olmo_core/distributed/parallel/context_parallel.py:11-305).

``cp2hp`` turns a sequence-sharded tensor ``[B, T/CP, H, D]`` into a head-sharded one ``[B, T, H/CP, D]``
so that ordinary attention can run over the full sequence; ``hp2cp`` is the inverse. On one NVSwitch box
every pair of GPUs has a direct full-bandwidth path, so the exchange is a single all-to-all whose
pack/unpack permutes are done once on each side -- or, with peer-mapped memory (``olmo_core_b200.parallel.ulysses``),
one kernel that stores every head group / sequence shard straight into its final place on the receiving GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ...config import Config
from ..nn import all_to_all_single

__all__ = [
    "ContextParallelConfig",
    "all_to_all_single_cp2hp",
    "all_to_all_cp2hp",
    "all_to_all_single_hp2cp",
    "all_to_all_hp2cp",
    "all_to_all_single_cp2hp_qkvpacked",
    "all_to_all_single_hp2cp_qkvpacked",
]


@dataclass
class ContextParallelConfig(Config):
    """The sequence dimension of every micro-batch is split over ``degree`` ranks."""

    degree: int


def _size(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def all_to_all_single_cp2hp(input_: torch.Tensor, cp_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[B, T/CP, H, D] -> [B, T, H/CP, D]``; a 3-D input ``[B, T/CP, H]`` is taken as ``D = 1``."""
    x, group = input_, cp_group
    cp = _size(group)
    if cp == 1:
        return x
    if x.dim() == 3:
        return all_to_all_single_cp2hp(x.unsqueeze(-1), group).squeeze(-1)
    B, t, H, D = x.shape
    if H % cp != 0:
        raise ValueError(f"number of heads ({H}) must be divisible by the context-parallel degree ({cp})")
    from ...parallel import ulysses

    if ulysses.peer_exchange_usable(x, group):
        return ulysses.cp2hp(x, group)
    # [B, t, cp, H/cp, D] -> [cp, B, t, H/cp, D]: slice r goes to rank r
    send = x.view(B, t, cp, H // cp, D).permute(2, 0, 1, 3, 4).contiguous()
    recv = all_to_all_single(group, send.view(cp * B * t, H // cp, D))
    # received chunk r holds sequence shard r
    return recv.view(cp, B, t, H // cp, D).permute(1, 0, 2, 3, 4).reshape(B, cp * t, H // cp, D)


def all_to_all_single_hp2cp(input_: torch.Tensor, cp_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[B, T, H/CP, D] -> [B, T/CP, H, D]``; a 3-D input ``[B, T, H/CP]`` is taken as ``D = 1``."""
    x, group = input_, cp_group
    cp = _size(group)
    if cp == 1:
        return x
    if x.dim() == 3:
        return all_to_all_single_hp2cp(x.unsqueeze(-1), group).squeeze(-1)
    B, T, h, D = x.shape
    if T % cp != 0:
        raise ValueError(f"sequence length ({T}) must be divisible by the context-parallel degree ({cp})")
    t = T // cp
    from ...parallel import ulysses

    if ulysses.peer_exchange_usable(x, group):
        return ulysses.hp2cp(x, group)
    send = x.view(B, cp, t, h, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = all_to_all_single(group, send.view(cp * B * t, h, D))
    # received chunk r holds head group r
    return recv.view(cp, B, t, h, D).permute(1, 2, 0, 3, 4).reshape(B, t, cp * h, D)


def all_to_all_cp2hp(inputs: List[torch.Tensor], cp_group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """Batched :func:`all_to_all_single_cp2hp`: tensors that share ``[B, T/CP, *, D]`` go in one exchange."""
    tensors, group = inputs, cp_group
    cp = _size(group)
    if any(t.dim() == 3 for t in tensors):  # mixed ranks: no common packing
        return [all_to_all_single_cp2hp(t, group) for t in tensors]
    from ...parallel import ulysses

    if cp == 1 or len(tensors) == 1 or ulysses.peer_exchange_usable(tensors[0], group):  # no packing for the peer kernel
        return [all_to_all_single_cp2hp(t, group) for t in tensors]
    heads = [t.shape[2] for t in tensors]
    packed = torch.cat([t.view(t.shape[0], t.shape[1], cp, h // cp, t.shape[3]) for t, h in zip(tensors, heads)], dim=3)
    B, t_, _, hsum, D = packed.shape
    out = all_to_all_single_cp2hp(packed.reshape(B, t_, cp * hsum, D), group)
    return list(out.split([h // cp for h in heads], dim=2))


def all_to_all_hp2cp(inputs: List[torch.Tensor], cp_group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """Batched :func:`all_to_all_single_hp2cp`."""
    tensors, group = inputs, cp_group
    cp = _size(group)
    if any(t.dim() == 3 for t in tensors):
        return [all_to_all_single_hp2cp(t, group) for t in tensors]
    from ...parallel import ulysses

    if cp == 1 or len(tensors) == 1 or ulysses.peer_exchange_usable(tensors[0], group):
        return [all_to_all_single_hp2cp(t, group) for t in tensors]
    local_heads = [t.shape[2] for t in tensors]
    packed = torch.cat(tensors, dim=2)
    out = all_to_all_single_hp2cp(packed, group)  # [B, t, cp*sum(h), D], rank-major
    B, t_, _, D = out.shape
    out = out.view(B, t_, cp, sum(local_heads), D)
    return [o.reshape(B, t_, cp * h, D) for o, h in zip(out.split(local_heads, dim=3), local_heads)]


def all_to_all_single_cp2hp_qkvpacked(input_: torch.Tensor, cp_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[B, T/CP, 3, H, D] -> [B, T, 3, H/CP, D]``"""
    qkv, group = input_, cp_group
    cp = _size(group)
    if cp == 1:
        return qkv
    B, t, three, H, D = qkv.shape
    x = qkv.view(B, t, three, cp, H // cp, D).permute(0, 1, 3, 2, 4, 5).reshape(B, t, cp * three * (H // cp), D)
    out = all_to_all_single_cp2hp(x, group)
    return out.view(B, cp * t, three, H // cp, D)


def all_to_all_single_hp2cp_qkvpacked(input_: torch.Tensor, cp_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[B, T, 3, H/CP, D] -> [B, T/CP, 3, H, D]``"""
    qkv, group = input_, cp_group
    cp = _size(group)
    if cp == 1:
        return qkv
    B, T, three, h, D = qkv.shape
    out = all_to_all_single_hp2cp(qkv.reshape(B, T, three * h, D), group)  # [B, t, cp*3*h, D]
    return out.view(B, T // cp, cp, three, h, D).permute(0, 1, 3, 2, 4, 5).reshape(B, T // cp, three, cp * h, D)
