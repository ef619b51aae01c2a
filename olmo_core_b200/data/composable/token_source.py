"""
Token and document sources (API of src/olmo_core/data/composable/token_source.py:37-677, sliced_token_source.py,
sampling_token_source.py, sampling_document_source.py, mixing_token_source.py, mixing_document_source.py).

A token source is an addressable sequence of token ids (optionally with a label mask); a document source also knows
where documents start and end. Every composite here (concatenation, slice, sample, mix) is the SAME data structure: a
list of pieces ``(child, start, end)`` with a prefix sum over their lengths, so that a token range is resolved with one
binary search and a walk over the pieces it touches.
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence, Tuple, TypedDict, Union

import numpy as np

from ...aliases import PathOrStr
from ..utils import get_rng
from .source_abc import SourceABC
from .utils import SEED_NOT_SET, as_ndarray, calculate_sample_sizes, resolve_seed

__all__ = [
    "TokenRange", "TokenSource", "DocumentSource", "InMemoryTokenSource", "InMemoryDocumentSource",
    "ConcatenatedTokenSource", "ConcatenatedDocumentSource", "SlicedTokenSource", "SamplingTokenSource",
    "SamplingDocumentSource", "MixingTokenSource", "MixingDocumentSource", "MixingTokenSourceSpec",
    "MixingDocumentSourceSpec",
]


class TokenRange(TypedDict, total=False):
    input_ids: np.ndarray
    label_mask: np.ndarray


class TokenSource(SourceABC):
    DISPLAY_ICON = ""

    def __len__(self) -> int:
        return self.num_tokens

    @abstractmethod
    def get_token_range(self, start_idx: int, end_idx: int) -> TokenRange:
        """Tokens ``[start_idx, end_idx)``."""
        raise NotImplementedError

    def __getitem__(self, key: Union[int, slice]) -> TokenRange:
        if isinstance(key, slice):
            if key.step not in (None, 1):
                raise IndexError("token sources only support contiguous slices")
            start, end, _ = key.indices(len(self))
            return self.get_token_range(start, end)
        if key < 0:
            key += len(self)
        return self.get_token_range(key, key + 1)

    def validate_indices(self, start_idx: int, end_idx: int) -> Tuple[int, int]:
        n = len(self)
        if start_idx < 0:
            start_idx += n
        if end_idx < 0:
            end_idx += n
        if not 0 <= start_idx <= end_idx <= n:
            raise IndexError(f"token range [{start_idx}, {end_idx}) is out of bounds for a source of {n} tokens")
        return start_idx, end_idx

    # -- composition ---------------------------------------------------------------------------------------
    def __add__(self, other: "TokenSource") -> "ConcatenatedTokenSource":
        if not isinstance(other, TokenSource):
            return NotImplemented
        return ConcatenatedTokenSource(self, other, work_dir=self.common_work_dir)

    def __mul__(self, factor: float) -> "SamplingTokenSource":
        return self.resize(factor)

    def sample(self, *, max_tokens: Optional[int] = None, factor: Optional[float] = None,
               seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSource":
        if (max_tokens is None) == (factor is None):
            raise ValueError("exactly one of 'max_tokens' and 'factor' is required")
        if max_tokens is None:
            max_tokens = int(factor * self.num_tokens)  # type: ignore[operator]
        return SamplingTokenSource(self, max_tokens=max_tokens, seed=seed, work_dir=self.common_work_dir, label=self.label)

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSource":
        """Shrink (``factor < 1``) or repeat (``factor > 1``) the source."""
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float) -> Tuple["SlicedTokenSource", "SlicedTokenSource"]:
        if not 0 < ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        cut = int(ratio * self.num_tokens)
        return (SlicedTokenSource(self, slice(0, cut), work_dir=self.common_work_dir, label=self.label),
                SlicedTokenSource(self, slice(cut, self.num_tokens), work_dir=self.common_work_dir, label=self.label))


class DocumentSource(TokenSource):
    @abstractmethod
    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        """``(start, end)`` of every document, in order, covering the source."""
        raise NotImplementedError

    def sample_by_docs(self, *, max_tokens: Optional[int] = None, factor: Optional[float] = None,
                       seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSource":
        if (max_tokens is None) == (factor is None):
            raise ValueError("exactly one of 'max_tokens' and 'factor' is required")
        if max_tokens is None:
            max_tokens = int(factor * self.num_tokens)  # type: ignore[operator]
        return SamplingDocumentSource(self, max_tokens=max_tokens, seed=seed, work_dir=self.common_work_dir,
                                      label=self.label)

    def resize_by_docs(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSource":
        return self.sample_by_docs(factor=factor, seed=seed)


# ------------------------------------------------------------------------------------------------------ leaves
class InMemoryTokenSource(TokenSource):
    def __init__(self, tokens: Sequence[int], *, work_dir: PathOrStr, label_mask: Optional[Sequence[bool]] = None,
                 label: Optional[str] = None):
        super().__init__(work_dir=work_dir, label=label)
        self._tokens = as_ndarray(tokens)
        self._mask = None if label_mask is None else as_ndarray(label_mask).astype(bool)
        if self._mask is not None and len(self._mask) != len(self._tokens):
            raise ValueError("'label_mask' must have one entry per token")

    @property
    def fingerprint(self) -> str:
        return self._hash(self._tokens.astype(np.int64).tobytes().hex()[:4096], len(self._tokens),
                          int(self._tokens.astype(np.int64).sum()), None if self._mask is None else int(self._mask.sum()))

    @property
    def num_tokens(self) -> int:
        return len(self._tokens)

    def get_token_range(self, start_idx: int, end_idx: int) -> TokenRange:
        start_idx, end_idx = self.validate_indices(start_idx, end_idx)
        out: TokenRange = {"input_ids": self._tokens[start_idx:end_idx]}
        if self._mask is not None:
            out["label_mask"] = self._mask[start_idx:end_idx]
        return out

    def children(self):
        return []


class InMemoryDocumentSource(InMemoryTokenSource, DocumentSource):
    """
    Documents end WITH the tokenizer's EOS token (where a BOS token exists, only an EOS followed by a BOS ends a
    document); whatever follows the last boundary is a document too
    (src/olmo_core/data/composable/token_source.py:292-354). ``eos_token_id`` / ``bos_token_id`` may be given instead of
    a tokenizer config.
    """

    def __init__(self, tokens: Sequence[int], *, tokenizer=None, work_dir: PathOrStr,
                 label_mask: Optional[Sequence[bool]] = None, label: Optional[str] = None,
                 eos_token_id: Optional[int] = None, bos_token_id: Optional[int] = None):
        super().__init__(tokens, work_dir=work_dir, label_mask=label_mask, label=label)
        if tokenizer is not None:
            eos_token_id, bos_token_id = tokenizer.eos_token_id, tokenizer.bos_token_id
        if eos_token_id is None:
            raise ValueError("a tokenizer config (or 'eos_token_id') is required")
        self._tokenizer = tokenizer
        self._eos, self._bos = eos_token_id, bos_token_id

    @property
    def eos_token_id(self) -> int:
        return self._eos

    @property
    def bos_token_id(self) -> Optional[int]:
        return self._bos

    @property
    def fingerprint(self) -> str:
        return self._hash(InMemoryTokenSource.fingerprint.fget(self), self._eos, self._bos)  # type: ignore[attr-defined]

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        n = len(self._tokens)
        if self._bos is None:
            ends = np.flatnonzero(self._tokens == self._eos) + 1
        else:
            ends = np.flatnonzero(np.logical_and(self._tokens[:-1] == self._eos, self._tokens[1:] == self._bos)) + 1
        start = 0
        for end in ends.tolist():
            yield start, end
            start = end
        if start != n:
            yield start, n


# ------------------------------------------------------------------------------------------------ composites
class _Spliced(TokenSource):
    """A sequence of pieces ``(child index, start, end)`` of child sources."""

    def __init__(self, children: Sequence[TokenSource], pieces: np.ndarray, *, work_dir: PathOrStr,
                 label: Optional[str] = None):
        super().__init__(work_dir=work_dir, label=label)
        self._children = tuple(children)
        self._pieces = np.asarray(pieces, dtype=np.int64).reshape(-1, 3)
        lengths = self._pieces[:, 2] - self._pieces[:, 1]
        if (lengths <= 0).any():
            self._pieces = self._pieces[lengths > 0]
            lengths = lengths[lengths > 0]
        self._ends = np.cumsum(lengths)

    @property
    def sources(self) -> Tuple[TokenSource, ...]:
        return self._children

    def children(self):
        return self._children

    @property
    def num_tokens(self) -> int:
        return int(self._ends[-1]) if len(self._ends) else 0

    @property
    def fingerprint(self) -> str:
        digest = int(np.bitwise_xor.reduce((self._pieces * np.array([1000003, 10007, 101])).sum(axis=1))) if len(self._pieces) else 0
        return self._hash(*[c.fingerprint for c in self._children], len(self._pieces), digest, self.num_tokens)

    def get_token_range(self, start_idx: int, end_idx: int) -> TokenRange:
        start_idx, end_idx = self.validate_indices(start_idx, end_idx)
        ids: List[np.ndarray] = []
        masks: List[np.ndarray] = []
        if end_idx > start_idx:
            i = int(np.searchsorted(self._ends, start_idx, side="right"))
            pos = start_idx
            while pos < end_idx:
                child, c_start, c_end = (int(v) for v in self._pieces[i])
                piece_begin = int(self._ends[i]) - (c_end - c_start)
                lo = c_start + (pos - piece_begin)
                hi = min(c_end, lo + (end_idx - pos))
                part = self._children[child].get_token_range(lo, hi)
                ids.append(as_ndarray(part["input_ids"]))
                if "label_mask" in part:
                    masks.append(as_ndarray(part["label_mask"]))
                pos += hi - lo
                i += 1
        out: TokenRange = {"input_ids": np.concatenate(ids) if ids else np.empty(0, dtype=np.int64)}
        if masks:
            if len(masks) != len(ids):
                raise RuntimeError("either every child source must provide a label mask or none")
            out["label_mask"] = np.concatenate(masks)
        return out


def _whole(children: Sequence[TokenSource]) -> np.ndarray:
    return np.array([(i, 0, c.num_tokens) for i, c in enumerate(children)], dtype=np.int64).reshape(-1, 3)


class ConcatenatedTokenSource(_Spliced):
    DISPLAY_ICON = ""

    def __init__(self, *sources: TokenSource, work_dir: PathOrStr, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        flat: List[TokenSource] = []
        for s in sources:  # nested concatenations are flattened
            flat.extend(s.sources if type(s) in (ConcatenatedTokenSource, ConcatenatedDocumentSource) else [s])
        super().__init__(flat, _whole(flat), work_dir=work_dir, label=label)


class ConcatenatedDocumentSource(ConcatenatedTokenSource, DocumentSource):
    def __init__(self, *sources: DocumentSource, work_dir: PathOrStr, label: Optional[str] = None):
        if not all(isinstance(s, DocumentSource) for s in sources):
            raise TypeError("every source must be a document source")
        super().__init__(*sources, work_dir=work_dir, label=label)

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        base = 0
        for child in self._children:
            for s, e in child.get_document_offsets():  # type: ignore[attr-defined]
                yield base + s, base + e
            base += child.num_tokens


class SlicedTokenSource(_Spliced):
    DISPLAY_ICON = ""

    def __init__(self, source: TokenSource, source_slice: slice, *, work_dir: PathOrStr, label: Optional[str] = None):
        if source_slice.step not in (None, 1):
            raise ValueError("only contiguous slices are supported")
        start, end, _ = source_slice.indices(source.num_tokens)
        self._slice = slice(start, end)
        super().__init__([source], np.array([[0, start, end]]), work_dir=work_dir, label=label)

    @property
    def source(self) -> TokenSource:
        return self._children[0]

    @property
    def source_slice(self) -> slice:
        return self._slice

    @property
    def slice_start(self) -> int:
        return self._slice.start

    @property
    def slice_stop(self) -> int:
        return self._slice.stop

    @property
    def slice_step(self) -> int:
        return 1


def _unwind(sources: Sequence[TokenSource]) -> List[TokenSource]:
    """
    Replace mixes by their per-source samples and samples by the pieces they are made of, breadth first (the order of
    src/olmo_core/data/composable/sampling_token_source.py:103-120), so that re-sampling keeps THEIR proportions.
    """
    from collections import deque

    out: List[TokenSource] = []
    frontier = deque(sources)
    while frontier:
        s = frontier.popleft()
        if isinstance(s, (MixingTokenSource, MixingDocumentSource)):
            frontier.extend(s.sampled_sources)
        elif type(s) is SamplingTokenSource:
            frontier.extend(s.sources)
        else:
            out.append(s)
    return out


class SamplingTokenSource(_Spliced):
    """
    ``max_tokens`` tokens drawn from the sources in proportion to their sizes, ignoring document boundaries: whole
    repetitions of a source first, then one contiguous window (at a random offset with a seed, at 0 without).
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: TokenSource, max_tokens: int, seed: Optional[int] = SEED_NOT_SET, work_dir: PathOrStr,
                 label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        if max_tokens <= 0:
            raise ValueError("'max_tokens' must be positive")
        self._seed = resolve_seed(seed)
        rng = None if self._seed is None else get_rng(self._seed)
        self.original_sources = tuple(sources)
        total = sum(s.num_tokens for s in sources)
        final: List[TokenSource] = []
        for leaf in _unwind(sources):
            want = round(max_tokens * (leaf.num_tokens / total))
            final.extend([leaf] * (want // leaf.num_tokens))
            rest = want % leaf.num_tokens
            if rest > 0:
                at = 0 if rng is None else int(rng.integers(0, leaf.num_tokens - rest))
                final.append(SlicedTokenSource(leaf, slice(at, at + rest), work_dir=work_dir))
        super().__init__(final, _whole(final), work_dir=work_dir, label=label)

    def children(self):
        return self.original_sources

    @property
    def seed(self) -> Optional[int]:
        return self._seed


class SamplingDocumentSource(_Spliced, DocumentSource):
    """
    Whole documents drawn from the (concatenated) sources: with a seed the documents are shuffled once; that order is
    repeated as often as it fits into ``max_tokens`` and followed by the longest prefix of it that fits into the rest
    (src/olmo_core/data/composable/sampling_document_source.py:87-170). Without a seed the natural order is used.
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: DocumentSource, max_tokens: int, seed: Optional[int] = SEED_NOT_SET,
                 work_dir: PathOrStr, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        if max_tokens <= 0:
            raise ValueError("'max_tokens' must be positive")
        self._seed = resolve_seed(seed)
        self._max_tokens = max_tokens
        self.original_sources = tuple(sources)
        source = ConcatenatedDocumentSource(*sources, work_dir=work_dir) if len(sources) > 1 else sources[0]
        self._source = source
        if self._seed is None:
            import warnings

            warnings.warn("No seed provided for SamplingDocumentSource. It's recommended to set a seed to ensure that the "
                          "distribution of documents in child sources are preserved.")
        offsets = np.fromiter((i for pair in source.get_document_offsets() for i in pair), dtype=np.uint64).reshape(-1, 2)
        if self._seed is not None:
            get_rng(self._seed).shuffle(offsets, axis=0)
        cumulative = np.cumsum(offsets[:, 1] - offsets[:, 0], dtype=np.uint64)
        total = int(cumulative[-1])
        picked = np.take(offsets, (cumulative <= max_tokens % total).nonzero()[0], axis=0)
        if max_tokens // total > 0:
            picked = np.concatenate([np.tile(offsets, (max_tokens // total, 1)), picked])
        if picked.shape[0] == 0:
            raise RuntimeError(f"Unable to sample {max_tokens} tokens from {source}")
        pieces = np.concatenate([np.zeros((len(picked), 1), dtype=np.int64), picked.astype(np.int64)], axis=1)
        super().__init__([source], pieces, work_dir=work_dir, label=label)

    def children(self):
        return self.original_sources

    @property
    def source(self) -> DocumentSource:
        return self._source

    @property
    def max_tokens(self) -> int:
        return self._max_tokens

    @property
    def seed(self) -> Optional[int]:
        return self._seed

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        starts = np.concatenate([[0], self._ends[:-1]])
        return zip(starts.tolist(), self._ends.tolist())


@dataclass
class MixingTokenSourceSpec:
    source: TokenSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None


@dataclass
class MixingDocumentSourceSpec:
    source: DocumentSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None


class MixingTokenSource(ConcatenatedTokenSource):
    """Sources combined at given ratios: each is sampled to the size the ratios call for, then concatenated."""

    DISPLAY_ICON = ""
    Spec = MixingTokenSourceSpec
    _by_docs = False

    def __init__(self, *source_specs, work_dir: PathOrStr, seed: Optional[int] = SEED_NOT_SET,
                 num_tokens: Optional[int] = None, label: Optional[str] = None):
        if not source_specs:
            raise ValueError("At least one source spec must be provided.")
        self._seed = resolve_seed(seed)
        labels = [spec.label or spec.source.label or str(i) for i, spec in enumerate(source_specs)]
        sizes = calculate_sample_sizes([spec.source.num_tokens for spec in source_specs],
                                       [spec.ratio for spec in source_specs],
                                       [spec.max_repetition_factor for spec in source_specs],
                                       target_size=num_tokens, labels=labels)
        sampled = []
        for i, (spec, size) in enumerate(zip(source_specs, sizes.tolist())):
            child_seed = None if self._seed is None else self._seed + i
            cls = SamplingDocumentSource if self._by_docs else SamplingTokenSource
            sampled.append(cls(spec.source, max_tokens=int(size), seed=child_seed, work_dir=work_dir, label=labels[i]))
        self.sampled_sources = tuple(sampled)
        _Spliced.__init__(self, sampled, _whole(sampled), work_dir=work_dir, label=label)

    @property
    def seed(self) -> Optional[int]:
        return self._seed


class MixingDocumentSource(MixingTokenSource, DocumentSource):
    Spec = MixingDocumentSourceSpec
    _by_docs = True

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        base = 0
        for child in self.sampled_sources:
            for s, e in child.get_document_offsets():
                yield base + s, base + e
            base += child.num_tokens


_CONFIG_NAMES = ('TokenSourceConfig', 'DocumentSourceConfig', 'ConcatenatedTokenSourceConfig', 'ConcatenatedDocumentSourceConfig', 'SplitTokenSourceConfig')


def __getattr__(name: str):
    # the config classes live in ``configs.py`` (which imports this module); they stay reachable under this module's name
    if name in _CONFIG_NAMES:
        from . import configs

        return getattr(configs, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
