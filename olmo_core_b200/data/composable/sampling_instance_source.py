"""Instance-level sampling of instance sources (src/olmo_core/data/composable/sampling_instance_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np

from ...aliases import PathOrStr
from ...exceptions import OLMoConfigurationError
from .instance_source import InstanceSource, InstanceSourceConfig, _Indexed
from .token_source import _default_seed
from .utils import SEED_NOT_SET, build_global_indices, resolve_seed

__all__ = ["SamplingInstanceSource", "SamplingInstanceSourceConfig"]


class SamplingInstanceSource(_Indexed):
    """
    ``max_instances`` (or ``max_tokens``) instances drawn from the sources in proportion to their sizes, in whole
    ``max_sequence_length`` units (src/olmo_core/data/composable/sampling_instance_source.py:62-234). Source ``i``
    contributes its instances in the order :func:`build_global_indices` gives for ``seed + i`` (its own order without a
    seed): that order repeated as often as it fits into the source's share, then its front.
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: InstanceSource, max_tokens: Optional[int] = None, max_instances: Optional[int] = None,
                 work_dir: PathOrStr, seed: Optional[int] = SEED_NOT_SET, label: Optional[str] = None):
        if not sources:
            raise OLMoConfigurationError("At least one source must be provided.")
        seq, max_seq = sources[0].sequence_length, sources[0].max_sequence_length
        if (max_tokens is None) == (max_instances is None):
            raise OLMoConfigurationError("Either max_tokens or max_instances must be set, but not both.")
        if max_instances is None:
            assert max_tokens is not None and max_tokens > 0
            max_instances = max_tokens // seq
        assert max_instances > 0
        self._max_instances = max_instances
        self._seed = resolve_seed(seed)
        if self._seed is None:
            import warnings

            warnings.warn("No seed provided for SamplingInstanceSource. It's recommended to set a seed to ensure that the "
                          "distribution of instances in child sources are preserved.")
        total = sum(len(src) for src in sources)
        group = max_seq // seq
        sizes, ids, idx = [], [], []
        for i, src in enumerate(sources):
            if src.sequence_length != seq or src.max_sequence_length != max_seq:
                raise OLMoConfigurationError("All sources must have the same sequence length and max sequence length.")
            size = group * (int(max_instances * (len(src) / total)) // group)
            sizes.append(size)
            order = build_global_indices(len(src), sequence_length=seq, max_sequence_length=max_seq,
                                         seed=None if self._seed is None else self._seed + i)
            picked = np.concatenate([np.tile(order, size // len(src)), order[: size % len(src)]]) if len(src) else order
            ids.append(np.full(len(picked), i, dtype=np.int32))
            idx.append(picked.astype(np.int64))
        self._source_sample_sizes = tuple(sizes)
        super().__init__(sources, np.concatenate(ids), np.concatenate(idx), work_dir=work_dir, label=label)

    @property
    def seed(self) -> Optional[int]:
        return self._seed

    @property
    def max_instances(self) -> int:
        return self._max_instances

    @property
    def source_sample_sizes(self) -> Tuple[int, ...]:
        return self._source_sample_sizes

    @property
    def num_instances(self) -> int:
        return sum(self._source_sample_sizes)


@dataclass
class SamplingInstanceSourceConfig(InstanceSourceConfig):
    sources: List[InstanceSourceConfig]
    max_tokens: Optional[int] = None
    max_instances: Optional[int] = None
    factor: Optional[float] = None
    seed: Optional[int] = field(default_factory=_default_seed)
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> SamplingInstanceSource:
        built = [s.build(work_dir) for s in self.sources]
        max_tokens, max_instances = self.max_tokens, self.max_instances
        if max_tokens is None and max_instances is None:
            assert self.factor is not None
            max_tokens = int(self.factor * sum(s.num_tokens for s in built))
        return SamplingInstanceSource(*built, max_tokens=max_tokens, max_instances=max_instances, seed=self.seed,
                                      work_dir=work_dir, label=self.label)


SamplingInstanceSource.Config = SamplingInstanceSourceConfig  # type: ignore[attr-defined]
