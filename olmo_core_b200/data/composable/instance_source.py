"""
Instance sources: fixed-length training instances cut from token sources, and composites of them
(API of src/olmo_core/data/composable/instance_source.py:25-432, concat_and_chunk_instance_source.py,
packing_instance_source.py, random_instance_source.py, sliced_instance_source.py, sampling_instance_source.py,
mixing_instance_source.py).

``max_sequence_length`` (a multiple of ``sequence_length``) is the unit in which leftover tokens are dropped: a source
offers the same text, in the same order, for every ``sequence_length`` that divides it.
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import Generator, Iterable, List, Optional, Sequence, Tuple, TypedDict

import numpy as np

from ...aliases import PathOrStr
from ..types import LongDocStrategy
from ..utils import InstancePacker, get_rng
from .source_abc import SourceABC
from .token_source import DocumentSource, TokenSource
from .utils import SEED_NOT_SET, as_ndarray, calculate_sample_sizes, resolve_seed

__all__ = [
    "Instance", "InstanceSource", "ConcatAndChunkInstanceSource", "PackingInstanceSource", "RandomInstanceSource",
    "ConcatenatedInstanceSource", "SlicedInstanceSource", "SamplingInstanceSource", "MixingInstanceSource",
    "MixingInstanceSourceSpec",
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
            max_instances = int(factor * len(self))
        return SamplingInstanceSource(self, max_tokens=max_tokens, max_instances=max_instances, seed=seed,
                                      work_dir=self.common_work_dir, label=self.label)

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingInstanceSource":
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float) -> Tuple["SlicedInstanceSource", "SlicedInstanceSource"]:
        """Two contiguous parts; the cut falls on a ``max_sequence_length`` boundary."""
        if not 0 < ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        group = self.max_sequence_length // self.sequence_length
        cut = int(ratio * len(self)) // group * group
        return (SlicedInstanceSource(self, slice(0, cut), work_dir=self.common_work_dir, label=self.label),
                SlicedInstanceSource(self, slice(cut, len(self)), work_dir=self.common_work_dir, label=self.label))

    def random_split(self, ratio: float, seed: Optional[int] = SEED_NOT_SET
                     ) -> Tuple["SamplingInstanceSource", "SamplingInstanceSource"]:
        """Two disjoint random parts."""
        if not 0 < ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        seed = resolve_seed(seed)
        order = np.arange(len(self)) if seed is None else get_rng(seed).permutation(len(self))
        cut = int(ratio * len(self))
        return tuple(SamplingInstanceSource(self, indices=np.sort(part), seed=seed, work_dir=self.common_work_dir,  # type: ignore[return-value]
                                            label=self.label) for part in (order[:cut], order[cut:]))

    def visualize(self, icons: bool = True) -> None:
        from .visualize import visualize_source

        visualize_source(self, icons=icons)


# ---------------------------------------------------------------------------------------------------- leaves
class ConcatAndChunkInstanceSource(InstanceSource):
    """Each token source is cut into consecutive instances; document boundaries are ignored."""

    DISPLAY_ICON = ""

    def __init__(self, *sources: TokenSource, sequence_length: int, max_sequence_length: Optional[int] = None,
                 work_dir: PathOrStr, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, max_sequence_length=max_sequence_length,
                         label=label)
        self._sources = tuple(sources)
        per_source = [s.num_tokens // self.max_sequence_length * (self.max_sequence_length // sequence_length)
                      for s in sources]
        self._ends = np.cumsum(per_source)

    @property
    def sources(self) -> Tuple[TokenSource, ...]:
        return self._sources

    def children(self):
        return self._sources

    @property
    def fingerprint(self) -> str:
        return self._hash(*[s.fingerprint for s in self._sources], self.sequence_length, self.max_sequence_length)

    def __len__(self) -> int:
        return int(self._ends[-1])

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        k = int(np.searchsorted(self._ends, idx, side="right"))
        local = idx - (int(self._ends[k - 1]) if k else 0)
        rng = self._sources[k].get_token_range(local * self.sequence_length, (local + 1) * self.sequence_length)
        out: Instance = {"input_ids": as_ndarray(rng["input_ids"])}
        if "label_mask" in rng:
            out["label_mask"] = as_ndarray(rng["label_mask"])
        return out


class PackingInstanceSource(InstanceSource):
    """
    Whole documents packed into instances with best-fit-decreasing bin packing; the tail of every instance is padding
    (masked out of the loss). Documents longer than an instance are truncated or split, per ``long_doc_strategy``.
    Sources are packed in groups of ``source_group_size`` so that instances rarely mix distant sources.
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: DocumentSource, sequence_length: int, pad_token_id: int, work_dir: PathOrStr,
                 max_sequence_length: Optional[int] = None, long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate,
                 source_group_size: int = 1, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        if max_sequence_length not in (None, sequence_length):
            raise ValueError("packed instances cannot be re-cut: 'max_sequence_length' must equal 'sequence_length'")
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, label=label)
        self._sources = tuple(sources)
        self._pad = pad_token_id
        self._strategy = LongDocStrategy(long_doc_strategy)
        self._group_size = source_group_size
        # instance -> rows of the document table; document table rows are (source index, start, end)
        self._docs = np.empty((0, 3), dtype=np.int64)
        self._instance_docs: List[List[int]] = []
        for g in range(0, len(sources), source_group_size):
            rows = []
            for i in range(g, min(g + source_group_size, len(sources))):
                for s, e in sources[i].get_document_offsets():
                    rows.extend(self._fit(i, s, e))
            table = np.array(rows, dtype=np.int64).reshape(-1, 3)
            packer = InstancePacker(sequence_length)
            instances, _, _ = packer.pack_documents(table[:, 1:])
            table = table[packer.last_order]  # the instances refer to the documents longest first
            base = len(self._docs)
            self._instance_docs.extend([[base + d for d in inst] for inst in instances])
            self._docs = np.concatenate([self._docs, table], axis=0)

    def _fit(self, source: int, start: int, end: int) -> List[Tuple[int, int, int]]:
        L = self.sequence_length
        if end - start <= L:
            return [(source, start, end)]
        if self._strategy == LongDocStrategy.truncate:
            return [(source, start, start + L)]
        return [(source, s, min(end, s + L)) for s in range(start, end, L)]

    def children(self):
        return self._sources

    @property
    def fingerprint(self) -> str:
        return self._hash(*[s.fingerprint for s in self._sources], self.sequence_length, self._pad, self._strategy,
                          self._group_size)

    def __len__(self) -> int:
        return len(self._instance_docs)

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        ids = np.full(self.sequence_length, self._pad, dtype=np.int64)
        mask = np.zeros(self.sequence_length, dtype=bool)
        pos = 0
        for d in self._instance_docs[idx]:
            src, s, e = (int(v) for v in self._docs[d])
            rng = self._sources[src].get_token_range(s, e)
            n = e - s
            ids[pos:pos + n] = as_ndarray(rng["input_ids"])
            mask[pos:pos + n] = as_ndarray(rng["label_mask"]) if "label_mask" in rng else True
            pos += n
        return {"input_ids": ids, "label_mask": mask}


class RandomInstanceSource(InstanceSource):
    """Uniformly random token ids, reproducible per index; for benchmarks and tests."""

    DISPLAY_ICON = ""

    def __init__(self, *, num_instances: int, sequence_length: int, vocab_size: int, work_dir: PathOrStr,
                 max_sequence_length: Optional[int] = None, seed: Optional[int] = SEED_NOT_SET, label: Optional[str] = None):
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, max_sequence_length=max_sequence_length,
                         label=label)
        self._n, self._vocab = num_instances, vocab_size
        self._seed = resolve_seed(seed) or 0

    def children(self):
        return []

    @property
    def fingerprint(self) -> str:
        return self._hash(self._n, self.sequence_length, self._vocab, self._seed)

    def __len__(self) -> int:
        return self._n

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        return {"input_ids": get_rng(self._seed + idx).integers(0, self._vocab, self.sequence_length, dtype=np.int64)}


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


class SlicedInstanceSource(_Indexed):
    DISPLAY_ICON = ""

    def __init__(self, source: InstanceSource, source_slice: slice, *, work_dir: PathOrStr, label: Optional[str] = None):
        idx = np.arange(len(source), dtype=np.int64)[source_slice]
        self.source_slice = source_slice
        super().__init__([source], np.zeros(len(idx), dtype=np.int32), idx, work_dir=work_dir, label=label)

    @property
    def source(self) -> InstanceSource:
        return self._children[0]


class SamplingInstanceSource(_Indexed):
    """
    ``max_instances`` (or ``max_tokens``) instances drawn from the sources in proportion to their sizes. Units of
    ``max_sequence_length // sequence_length`` neighbouring instances are kept together. A source smaller than its
    share is repeated whole before the remainder is drawn (at random with a seed, from the front without).
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: InstanceSource, max_tokens: Optional[int] = None, max_instances: Optional[int] = None,
                 indices: Optional[np.ndarray] = None, seed: Optional[int] = SEED_NOT_SET, work_dir: PathOrStr,
                 label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        self._seed = resolve_seed(seed)
        if indices is not None:  # explicit selection from a single source (used by random_split)
            assert len(sources) == 1
            super().__init__(sources, np.zeros(len(indices), dtype=np.int32), indices, work_dir=work_dir, label=label)
            return
        seq, max_seq = sources[0].sequence_length, sources[0].max_sequence_length
        if (max_tokens is None) == (max_instances is None):
            raise ValueError("exactly one of 'max_tokens' and 'max_instances' is required")
        if max_instances is None:
            max_instances = max_tokens // seq  # type: ignore[operator]
        group = max_seq // seq
        total = sum(len(s) for s in sources)
        rng = None if self._seed is None else get_rng(self._seed)
        ids, idx = [], []
        for i, s in enumerate(sources):
            units_available = len(s) // group
            units_wanted = round(max_instances * len(s) / total) // group
            if units_available == 0 or units_wanted == 0:
                continue
            picked = [np.arange(units_available)] * (units_wanted // units_available)
            rest = units_wanted % units_available
            if rest:
                picked.append(np.arange(rest) if rng is None else np.sort(rng.choice(units_available, rest, replace=False)))
            units = np.concatenate(picked)
            inst = (units[:, None] * group + np.arange(group)[None, :]).reshape(-1)
            ids.append(np.full(len(inst), i, dtype=np.int32))
            idx.append(inst)
        super().__init__(sources, np.concatenate(ids) if ids else np.empty(0, np.int32),
                         np.concatenate(idx) if idx else np.empty(0, np.int64), work_dir=work_dir, label=label)

    @property
    def seed(self) -> Optional[int]:
        return self._seed


@dataclass
class MixingInstanceSourceSpec:
    source: InstanceSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None


class MixingInstanceSource(_Indexed):
    """Instance sources combined at given ratios; ``num_tokens`` / ``num_instances`` fixes the size of the mix."""

    DISPLAY_ICON = ""
    Spec = MixingInstanceSourceSpec

    def __init__(self, *source_specs: MixingInstanceSourceSpec, work_dir: PathOrStr, seed: Optional[int] = SEED_NOT_SET,
                 num_tokens: Optional[int] = None, num_instances: Optional[int] = None, label: Optional[str] = None):
        if not source_specs:
            raise ValueError("At least one source spec must be provided.")
        self._seed = resolve_seed(seed)
        seq = source_specs[0].source.sequence_length
        if num_tokens is not None and num_instances is None:
            num_instances = num_tokens // seq
        labels = [spec.label or spec.source.label or str(i) for i, spec in enumerate(source_specs)]
        sizes = calculate_sample_sizes([len(spec.source) for spec in source_specs], [spec.ratio for spec in source_specs],
                                       [spec.max_repetition_factor for spec in source_specs], target_size=num_instances,
                                       labels=labels, unit="instances")
        sampled = [SamplingInstanceSource(spec.source, max_instances=int(size),
                                          seed=None if self._seed is None else self._seed + i, work_dir=work_dir,
                                          label=labels[i])
                   for i, (spec, size) in enumerate(zip(source_specs, sizes.tolist()))]
        self.sampled_sources = tuple(sampled)
        super().__init__(sampled, *_all_of(sampled), work_dir=work_dir, label=label)

    @property
    def seed(self) -> Optional[int]:
        return self._seed


_CONFIG_NAMES = ('InstanceSourceConfig', 'ConcatenatedInstanceSourceConfig', 'SplitInstanceSourceConfig')


def __getattr__(name: str):
    # the config classes live in ``configs.py`` (which imports this module); they stay reachable under this module's name
    if name in _CONFIG_NAMES:
        from . import configs

        return getattr(configs, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
