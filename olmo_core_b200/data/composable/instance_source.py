"""
Instance sources: fixed-length training instances cut from token sources, their composites and the bases of their
configs (API of src/olmo_core/data/composable/instance_source.py:25-432). The concrete sources live in the modules named
after them.

``max_sequence_length`` (a multiple of ``sequence_length``) is the unit in which leftover tokens are dropped: a source
offers the same text, in the same order, for every ``sequence_length`` that divides it.
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import TYPE_CHECKING, Generator, List, Optional, Sequence, Tuple, TypedDict

import numpy as np

from ...aliases import PathOrStr
from ...config import Config
from .source_abc import SourceABC
from .utils import SEED_NOT_SET, resolve_seed

if TYPE_CHECKING:
    from .sampling_instance_source import SamplingInstanceSource, SamplingInstanceSourceConfig
    from .sliced_instance_source import SlicedInstanceSource

__all__ = [
    "Instance", "InstanceSource", "ConcatenatedInstanceSource", "InstanceSourceConfig",
    "ConcatenatedInstanceSourceConfig", "SplitInstanceSourceConfig",
]


class Instance(TypedDict, total=False):
    input_ids: np.ndarray
    label_mask: np.ndarray


class InstanceSource(SourceABC):
    DISPLAY_ICON = ""

    def __init__(self, *, work_dir: PathOrStr, sequence_length: int, max_sequence_length: Optional[int] = None,
                 label: Optional[str] = None):
        super().__init__(work_dir=work_dir, label=label)
        max_sequence_length = max_sequence_length or sequence_length
        if max_sequence_length % sequence_length != 0:
            raise ValueError("'max_sequence_length' must be a multiple of 'sequence_length'")
        self._sequence_length, self._max_sequence_length = sequence_length, max_sequence_length

    @property
    def sequence_length(self) -> int:
        return self._sequence_length

    @property
    def max_sequence_length(self) -> int:
        return self._max_sequence_length

    @property
    def num_tokens(self) -> int:
        return len(self) * self.sequence_length

    @abstractmethod
    def __len__(self) -> int:
        raise NotImplementedError

    @abstractmethod
    def __getitem__(self, idx: int) -> Instance:
        raise NotImplementedError

    def __iter__(self) -> Generator[Instance, None, None]:
        for i in range(len(self)):
            yield self[i]

    def validate_index(self, idx: int) -> int:
        n = len(self)
        if idx < 0:
            idx += n
        if not 0 <= idx < n:
            raise IndexError(f"index {idx} is out of bounds for a source of {n} instances")
        return idx

    # -- composition ---------------------------------------------------------------------------------------
    def __add__(self, other: "InstanceSource") -> "ConcatenatedInstanceSource":
        if not isinstance(other, InstanceSource):
            return NotImplemented
        return ConcatenatedInstanceSource(self, other, work_dir=self.common_work_dir)

    def __mul__(self, factor: float) -> "SamplingInstanceSource":
        return self.resize(factor)

    def sample(self, *, max_tokens: Optional[int] = None, max_instances: Optional[int] = None,
               factor: Optional[float] = None, seed: Optional[int] = SEED_NOT_SET) -> "SamplingInstanceSource":
        given = [x is not None for x in (max_tokens, max_instances, factor)]
        if sum(given) != 1:
            raise ValueError("exactly one of 'max_tokens', 'max_instances' and 'factor' is required")
        if factor is not None:
            max_tokens = int(self.num_tokens * factor)
        from .sampling_instance_source import SamplingInstanceSource

        return SamplingInstanceSource(self, max_tokens=max_tokens, max_instances=max_instances, seed=seed,
                                      work_dir=self.common_work_dir, label=self.label)

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingInstanceSource":
        assert factor > 0
        return self.sample(max_tokens=int(self.num_tokens * factor), seed=seed)

    def split(self, ratio: float, seed: Optional[int] = None) -> Tuple["SlicedInstanceSource", "SlicedInstanceSource"]:
        """
        Two disjoint parts holding ``ratio`` and ``1 - ratio`` of the instances; the cut falls on a
        ``max_sequence_length`` boundary. With a ``seed`` the instances are dealt to the parts at random (in units of
        ``max_sequence_length``), without one the first part is the front of the source
        (src/olmo_core/data/composable/instance_source.py:179-204).
        """
        if not 0 < ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        from .sliced_instance_source import SlicedInstanceSource

        cut = int(((ratio * self.num_tokens) // self.max_sequence_length) * (self.max_sequence_length // self.sequence_length))
        return (SlicedInstanceSource(self, slice(0, cut), seed=seed, work_dir=self.common_work_dir),
                SlicedInstanceSource(self, slice(cut, None), seed=seed, work_dir=self.common_work_dir))

    def random_split(self, ratio: float, seed: Optional[int] = SEED_NOT_SET
                     ) -> Tuple["SlicedInstanceSource", "SlicedInstanceSource"]:
        """:meth:`split` with a (by default fresh) seed."""
        return self.split(ratio, seed=seed)

    def visualize(self, icons: bool = True) -> None:
        from .visualize import visualize_source

        visualize_source(self, icons=icons)



# ------------------------------------------------------------------------------------------------ composites
class _Indexed(InstanceSource):
    """Instances addressed through a table ``(child, index in child)``."""

    def __init__(self, children: Sequence[InstanceSource], child_ids: np.ndarray, child_idx: np.ndarray, *,
                 work_dir: PathOrStr, label: Optional[str] = None):
        seqs = {(c.sequence_length, c.max_sequence_length) for c in children}
        if len(seqs) != 1:
            raise ValueError("all sources must share 'sequence_length' and 'max_sequence_length'")
        (seq, max_seq), = seqs
        super().__init__(work_dir=work_dir, sequence_length=seq, max_sequence_length=max_seq, label=label)
        self._children = tuple(children)
        self._child_ids = np.asarray(child_ids, dtype=np.int32)
        self._child_idx = np.asarray(child_idx, dtype=np.int64)

    @property
    def sources(self) -> Tuple[InstanceSource, ...]:
        return self._children

    def children(self):
        return self._children

    @property
    def fingerprint(self) -> str:
        digest = int((self._child_idx * 2654435761 % 4294967291).sum()) if len(self._child_idx) else 0
        return self._hash(*[c.fingerprint for c in self._children], len(self._child_idx), digest)

    def __len__(self) -> int:
        return len(self._child_idx)

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        return self._children[int(self._child_ids[idx])][int(self._child_idx[idx])]


def _all_of(children: Sequence[InstanceSource]) -> Tuple[np.ndarray, np.ndarray]:
    ids = np.concatenate([np.full(len(c), i, dtype=np.int32) for i, c in enumerate(children)])
    idx = np.concatenate([np.arange(len(c), dtype=np.int64) for c in children])
    return ids, idx


class ConcatenatedInstanceSource(_Indexed):
    DISPLAY_ICON = ""

    def __init__(self, *sources: InstanceSource, work_dir: PathOrStr, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        super().__init__(sources, *_all_of(sources), work_dir=work_dir, label=label)


# ----------------------------------------------------------------------------------------------------- configs
@dataclass
class InstanceSourceConfig(Config):
    def build(self, work_dir: PathOrStr) -> InstanceSource:
        raise NotImplementedError

    def __add__(self, other: "InstanceSourceConfig") -> "ConcatenatedInstanceSourceConfig":
        return ConcatenatedInstanceSourceConfig(sources=[self, other])

    def __mul__(self, factor: float) -> "SamplingInstanceSourceConfig":
        return self.resize(factor)

    def sample(self, *, max_tokens: Optional[int] = None, max_instances: Optional[int] = None,
               factor: Optional[float] = None, seed: Optional[int] = SEED_NOT_SET) -> "SamplingInstanceSourceConfig":
        from .sampling_instance_source import SamplingInstanceSourceConfig

        return SamplingInstanceSourceConfig(sources=[self], max_tokens=max_tokens, max_instances=max_instances,
                                            factor=factor, seed=resolve_seed(seed))

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingInstanceSourceConfig":
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float, seed: Optional[int] = None
              ) -> Tuple["SplitInstanceSourceConfig", "SplitInstanceSourceConfig"]:
        """Two disjoint parts (``ratio`` / ``1 - ratio`` of the instances); a ``seed`` deals the instances at random."""
        seed = resolve_seed(seed)
        return (SplitInstanceSourceConfig(source=self, ratio=ratio, idx=0, seed=seed),
                SplitInstanceSourceConfig(source=self, ratio=ratio, idx=1, seed=seed))

    def random_split(self, ratio: float, seed: Optional[int] = SEED_NOT_SET
                     ) -> Tuple["SplitInstanceSourceConfig", "SplitInstanceSourceConfig"]:
        return self.split(ratio, seed=seed)


@dataclass
class ConcatenatedInstanceSourceConfig(InstanceSourceConfig):
    sources: List[InstanceSourceConfig]
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> ConcatenatedInstanceSource:
        return ConcatenatedInstanceSource(*[s.build(work_dir) for s in self.sources], work_dir=work_dir, label=self.label)


@dataclass
class SplitInstanceSourceConfig(InstanceSourceConfig):
    source: InstanceSourceConfig
    ratio: float
    idx: int
    seed: Optional[int] = None

    def __post_init__(self):
        if not 0 < self.ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        if self.idx not in (0, 1):
            raise ValueError("'idx' must be 0 or 1")
        self.seed = resolve_seed(self.seed)

    def build(self, work_dir: PathOrStr) -> InstanceSource:
        return self.source.build(work_dir).split(self.ratio, seed=self.seed)[self.idx]


ConcatenatedInstanceSource.Config = ConcatenatedInstanceSourceConfig  # type: ignore[attr-defined]
