"""Caches ``DeviceMesh.__getitem__`` (sub-mesh creation is slow and called on hot paths) (monkey_patcher.py:10-23)."""

from dataclasses import dataclass
from functools import lru_cache

from .callback import Callback

__all__ = ["MonkeyPatcherCallback"]


@dataclass
class MonkeyPatcherCallback(Callback):
    def pre_train(self) -> None:
        from torch.distributed.device_mesh import DeviceMesh

        if not getattr(DeviceMesh.__getitem__, "_ocb_cached", False):
            cached = lru_cache(maxsize=None)(DeviceMesh.__getitem__)
            cached._ocb_cached = True  # type: ignore[attr-defined]
            DeviceMesh.__getitem__ = cached  # type: ignore[method-assign]
