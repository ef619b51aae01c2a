"""A slice of an instance source (src/olmo_core/data/composable/sliced_instance_source.py)."""

from __future__ import annotations

from typing import Optional

import numpy as np

from ...aliases import PathOrStr
from ...exceptions import OLMoConfigurationError
from .instance_source import InstanceSource, SplitInstanceSourceConfig, _Indexed
from .utils import build_global_indices, resolve_seed

__all__ = ["SlicedInstanceSource"]


class SlicedInstanceSource(_Indexed):
    """
    A slice of the source's instances in the order :func:`build_global_indices` gives for ``seed`` (the source's own
    order without one); whole ``max_sequence_length`` units only (src/olmo_core/data/composable/sliced_instance_source.py).
    """

    DISPLAY_ICON = ""

    def __init__(self, source: InstanceSource, source_slice: slice, *, seed: Optional[int] = None, work_dir: PathOrStr,
                 label: Optional[str] = None):
        self._slice = source_slice
        self._seed = resolve_seed(seed)
        order = build_global_indices(len(source), sequence_length=source.sequence_length,
                                     max_sequence_length=source.max_sequence_length, seed=self._seed)[source_slice]
        if order.size == 0:
            raise OLMoConfigurationError(f"{type(self).__name__} created with an empty slice ({source_slice}) from source "
                                         f"with {len(source):,d} instances.")
        group = source.max_sequence_length // source.sequence_length
        order = order[: group * (len(order) // group)]
        super().__init__([source], np.zeros(len(order), dtype=np.int32), order.astype(np.int64), work_dir=work_dir,
                         label=label if label is not None else source.label)

    @property
    def source(self) -> InstanceSource:
        return self._children[0]

    @property
    def source_slice(self) -> slice:
        return self._slice

    @property
    def seed(self) -> Optional[int]:
        return self._seed

    @property
    def num_instances(self) -> int:
        return len(self)

    @property
    def fingerprint(self) -> str:
        group = self.max_sequence_length // self.sequence_length
        sl = self._slice
        return self._hash(type(self).__name__, self._seed, self.max_sequence_length,
                          (sl.start // group) if sl.start is not None else 0, (sl.stop // group) if sl.stop is not None else -1,
                          (sl.step // group) if sl.step is not None else 1, self.source.fingerprint)


SlicedInstanceSource.Config = SplitInstanceSourceConfig  # type: ignore[attr-defined]
