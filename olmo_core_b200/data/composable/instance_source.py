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
from ...exceptions import OLMoConfigurationError
from .utils import SEED_NOT_SET, as_ndarray, build_global_indices, calculate_sample_sizes, resolve_seed

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
            max_tokens = int(self.num_tokens * factor)
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

    def __init__(self, *sources: DocumentSource, sequence_length: int, work_dir: PathOrStr, tokenizer=None,
                 pad_token_id: Optional[int] = None, max_sequence_length: Optional[int] = None,
                 long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate, source_group_size: int = 1,
                 label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        if tokenizer is not None:
            pad_token_id = tokenizer.pad_token_id
        if pad_token_id is None:
            raise ValueError("a tokenizer config (or 'pad_token_id') is required")
        self._tokenizer = tokenizer
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
    def sources(self) -> Tuple[DocumentSource, ...]:
        return self._sources

    @property
    def source_groups(self) -> Tuple[Tuple[DocumentSource, ...], ...]:
        return tuple(self._sources[g:g + self._group_size] for g in range(0, len(self._sources), self._group_size))

    @property
    def source_group_size(self) -> int:
        return self._group_size

    @property
    def long_doc_strategy(self) -> LongDocStrategy:
        return self._strategy

    @property
    def pad_token_id(self) -> int:
        return self._pad

    @property
    def num_instances(self) -> int:
        return len(self._instance_docs)

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
    """
    Random token ids with random document boundaries, reproducible per index: for benchmarks and tests
    (src/olmo_core/data/composable/random_instance_source.py:44-196). Special tokens never appear inside a document;
    every ``max_sequence_length`` window ends with EOS (and starts with BOS when the tokenizer has one) and holds about
    ``max_sequence_length / avg_document_length`` documents.
    """

    DISPLAY_ICON = ""

    def __init__(self, *, tokenizer=None, sequence_length: int, avg_document_length: Optional[int] = None,
                 seed: Optional[int] = SEED_NOT_SET, num_instances: Optional[int] = None, num_tokens: Optional[int] = None,
                 max_sequence_length: Optional[int] = None, label: Optional[str] = None, work_dir: PathOrStr,
                 vocab_size: Optional[int] = None):
        if (num_tokens is None) == (num_instances is None):
            raise ValueError("Either num_tokens or num_instances must be set, but not both.")
        if num_tokens is None:
            num_tokens = num_instances * sequence_length  # type: ignore[operator]
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, max_sequence_length=max_sequence_length,
                         label=label)
        if tokenizer is None:
            if vocab_size is None:
                raise ValueError("a tokenizer config (or 'vocab_size') is required")
            from ..tokenizer import TokenizerConfig

            tokenizer = TokenizerConfig(vocab_size=vocab_size, eos_token_id=0, pad_token_id=1)
        self._tokenizer = tokenizer
        self._num_tokens = self.max_sequence_length * (num_tokens // self.max_sequence_length)
        self._avg_document_length = avg_document_length or self.max_sequence_length
        seed = resolve_seed(seed)
        assert seed is not None
        self._seed = seed

    @property
    def num_tokens(self) -> int:
        return self._num_tokens

    @property
    def seed(self) -> int:
        return self._seed

    @property
    def eos_token_id(self) -> int:
        return self._tokenizer.eos_token_id

    @property
    def bos_token_id(self) -> Optional[int]:
        return self._tokenizer.bos_token_id

    @property
    def pad_token_id(self) -> int:
        return self._tokenizer.pad_token_id

    @property
    def vocab_size(self) -> int:
        return self._tokenizer.vocab_size

    @property
    def avg_document_length(self) -> int:
        return self._avg_document_length

    @property
    def non_special_token(self) -> int:
        special = (self.eos_token_id, self.bos_token_id, self.pad_token_id)
        for token_id in range(self.vocab_size):
            if token_id not in special:
                return token_id
        raise RuntimeError("No non-special token found in the vocabulary.")

    @property
    def dtype(self):
        for dtype in (np.uint8, np.uint16, np.uint32):
            if np.iinfo(dtype).max >= self.vocab_size:
                return dtype
        return np.uint64

    def children(self):
        return []

    @property
    def fingerprint(self) -> str:
        return self._hash(self._num_tokens, self._seed, self.max_sequence_length, self.eos_token_id, self.bos_token_id,
                          self.pad_token_id, self.vocab_size)

    def __len__(self) -> int:
        return self._num_tokens // self.sequence_length

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        per_window = self.max_sequence_length // self.sequence_length
        window = idx // per_window
        rng = get_rng(self._seed + window)
        L = self.max_sequence_length
        tokens = rng.integers(0, self.vocab_size, L, dtype=self.dtype)
        filler = self.non_special_token
        for special in (self.eos_token_id, self.pad_token_id, self.bos_token_id):
            if special is not None:
                tokens[tokens == special] = filler
        num_docs = max(1, round(rng.integers(-3, 3) + L / self._avg_document_length))
        tokens[-1] = self.eos_token_id
        if self.bos_token_id is not None:
            tokens[0] = self.bos_token_id
        if num_docs > 1:
            margin = 1 if self.bos_token_id is None else 2
            ends = margin + rng.permutation(L - 2 * margin - 1)[: num_docs - 1]
            tokens[ends] = self.eos_token_id
            if self.bos_token_id is not None:
                tokens[ends + 1] = self.bos_token_id
        if per_window > 1:
            start = (idx % per_window) * self.sequence_length
            tokens = tokens[start: start + self.sequence_length]
        return {"input_ids": tokens}


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
class MixingInstanceSourceSpec:
    source: InstanceSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None

    def __post_init__(self):
        if self.ratio <= 0:
            raise OLMoConfigurationError("Ratio must be greater than 0.")
        if self.max_repetition_factor < 1.0:
            raise OLMoConfigurationError("Max repetition must be at least 1.0.")


class MixingInstanceSource(_Indexed):
    """
    Instance sources combined at given ratios (src/olmo_core/data/composable/mixing_instance_source.py:111-245): the
    shares are worked out in tokens, every source is then sampled with :class:`SamplingInstanceSource` (seed ``seed + i``)
    and the samples are concatenated. ``num_tokens`` / ``num_instances`` fixes the size of the mix.
    """

    DISPLAY_ICON = ""
    Spec = MixingInstanceSourceSpec

    def __init__(self, *source_specs: MixingInstanceSourceSpec, work_dir: PathOrStr, seed: Optional[int] = SEED_NOT_SET,
                 label: Optional[str] = None, num_tokens: Optional[int] = None, num_instances: Optional[int] = None):
        if not source_specs:
            raise OLMoConfigurationError("At least one source spec must be provided.")
        self._seed = resolve_seed(seed)
        seq = source_specs[0].source.sequence_length
        if num_tokens is not None and num_instances is not None and num_tokens != num_instances * seq:
            raise OLMoConfigurationError("`num_tokens` and `num_instances` are mutually exclusive")
        if num_instances is not None:
            num_tokens = num_instances * seq
        labels = [spec.label or spec.source.label or str(i) for i, spec in enumerate(source_specs)]
        sizes = calculate_sample_sizes([spec.source.num_tokens for spec in source_specs], [spec.ratio for spec in source_specs],
                                       [spec.max_repetition_factor for spec in source_specs], target_size=num_tokens,
                                       labels=labels)
        sampled = [SamplingInstanceSource(spec.source, max_tokens=int(size),
                                          seed=None if self._seed is None else self._seed + i, work_dir=work_dir,
                                          label=spec.label or spec.source.label)
                   for i, (spec, size) in enumerate(zip(source_specs, sizes.tolist()))]
        self._sampled_sources = tuple(sampled)
        super().__init__(sampled, *_all_of(sampled), work_dir=work_dir, label=label)

    @property
    def sampled_sources(self) -> Tuple[SamplingInstanceSource, ...]:
        return self._sampled_sources

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
