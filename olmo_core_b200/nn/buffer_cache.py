"""
Namespaced cache for non-persistent buffers that several modules share, e.g. the RoPE sin/cos tables of
all layers (src/olmo_core/nn/buffer_cache.py:10-60). Buffers kept here do not show up in
``state_dict()`` and are not touched by parameter sharding.
"""

from __future__ import annotations

from collections.abc import MutableMapping
from typing import Dict, Iterator, Optional

import torch

__all__ = ["BufferCache"]


class BufferCache(MutableMapping):
    def __init__(self, namespace: str = "", store: Optional[Dict[str, torch.Tensor]] = None):
        self._namespace = namespace
        self._store: Dict[str, torch.Tensor] = {} if store is None else store

    def _key(self, key: str) -> str:
        return f"{self._namespace}.{key}" if self._namespace else key

    def __getitem__(self, key: str) -> torch.Tensor:
        return self._store[self._key(key)]

    def __setitem__(self, key: str, value: torch.Tensor) -> None:
        self._store[self._key(key)] = value

    def __delitem__(self, key: str) -> None:
        del self._store[self._key(key)]

    def __iter__(self) -> Iterator[str]:
        prefix = self._namespace + "." if self._namespace else ""
        for k in self._store:
            if k.startswith(prefix):
                yield k[len(prefix):]

    def __len__(self) -> int:
        return sum(1 for _ in self)

    def get_for_device(self, key: str, device: torch.device) -> Optional[torch.Tensor]:
        """The cached tensor, moved to (and re-cached on) ``device``; ``None`` when absent."""
        tensor = self.get(key)
        if tensor is None:
            return None
        if tensor.device != torch.device(device):
            tensor = tensor.to(device, non_blocking=True)
            self[key] = tensor
        return tensor

    def with_namespace(self, namespace: str) -> "BufferCache":
        """A view on the same storage under a sub-namespace."""
        return BufferCache(self._key(namespace), self._store)
