"""
Token and document sources and the bases of their configs
(API of src/olmo_core/data/composable/token_source.py:37-677).

A token source is an addressable sequence of token ids (optionally with a label mask); a document source also knows
where documents start and end. Every composite (concatenation here; slice, sample and mix in the modules named after
them) is the SAME data structure: a list of pieces ``(child, start, end)`` with a prefix sum over their lengths, so that
a token range is resolved with one binary search and a walk over the pieces it touches.

Every source class has its serializable config at ``<Source>.Config``. Token-source configs ``build(work_dir)`` into a
LIST of sources (a glob may expand into many).
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import TYPE_CHECKING, Any, Iterable, List, Optional, Sequence, Tuple, TypedDict, Union

import numpy as np

from ...aliases import PathOrStr
from ...config import Config
from .source_abc import SourceABC
from .utils import SEED_NOT_SET, as_ndarray, resolve_seed

if TYPE_CHECKING:
    from .sampling_document_source import SamplingDocumentSource, SamplingDocumentSourceConfig
    from .sampling_token_source import SamplingTokenSource, SamplingTokenSourceConfig
    from .sliced_token_source import SlicedTokenSource

__all__ = [
    "TokenRange", "TokenSource", "DocumentSource", "InMemoryTokenSource", "InMemoryDocumentSource",
    "ConcatenatedTokenSource", "ConcatenatedDocumentSource", "TokenSourceConfig", "DocumentSourceConfig",
    "ConcatenatedTokenSourceConfig", "ConcatenatedDocumentSourceConfig", "SplitTokenSourceConfig",
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
        from .sampling_token_source import SamplingTokenSource

        return SamplingTokenSource(self, max_tokens=max_tokens, seed=seed, work_dir=self.common_work_dir, label=self.label)

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSource":
        """Shrink (``factor < 1``) or repeat (``factor > 1``) the source."""
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float) -> Tuple["SlicedTokenSource", "SlicedTokenSource"]:
        if not 0 < ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        from .sliced_token_source import SlicedTokenSource

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
        from .sampling_document_source import SamplingDocumentSource

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



# ----------------------------------------------------------------------------------------------------- configs
@dataclass
class TokenSourceConfig(Config):
    def build(self, work_dir: PathOrStr) -> List["TokenSource"]:
        raise NotImplementedError

    def __add__(self, other: "TokenSourceConfig") -> "TokenSourceConfig":
        """Concatenation; two document sources give a document source."""
        if isinstance(self, DocumentSourceConfig) and isinstance(other, DocumentSourceConfig):
            return ConcatenatedDocumentSourceConfig(sources=[self, other])
        if isinstance(other, TokenSourceConfig):
            return ConcatenatedTokenSourceConfig(sources=[self, other])
        raise TypeError(f"Cannot add {type(self)} with {type(other)}.")

    def __mul__(self, factor: float) -> "SamplingTokenSourceConfig":
        if not isinstance(factor, (float, int)):
            raise TypeError(f"Cannot multiply {type(self)} with {type(factor)}.")
        return self.resize(factor)

    def sample(self, *, max_tokens: Optional[int] = None, factor: Optional[float] = None,
               seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSourceConfig":
        from .sampling_token_source import SamplingTokenSourceConfig

        return SamplingTokenSourceConfig(sources=[self], max_tokens=max_tokens, factor=factor, seed=resolve_seed(seed))

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSourceConfig":
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float) -> Tuple["SplitTokenSourceConfig", "SplitTokenSourceConfig"]:
        return (SplitTokenSourceConfig(source=self, ratio=ratio, idx=0), SplitTokenSourceConfig(source=self, ratio=ratio, idx=1))


@dataclass
class DocumentSourceConfig(TokenSourceConfig):
    def build(self, work_dir: PathOrStr) -> List["DocumentSource"]:  # type: ignore[override]
        raise NotImplementedError

    def sample_by_docs(self, *, max_tokens: Optional[int] = None, factor: Optional[float] = None,
                       seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSourceConfig":
        from .sampling_document_source import SamplingDocumentSourceConfig

        return SamplingDocumentSourceConfig(sources=[self], max_tokens=max_tokens, factor=factor, seed=resolve_seed(seed))

    def resize_by_docs(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSourceConfig":
        return self.sample_by_docs(factor=factor, seed=seed)


def _default_seed() -> int:
    return resolve_seed(SEED_NOT_SET)


def _build_all(configs: List[Any], work_dir: PathOrStr) -> List[Any]:
    out: List[Any] = []
    for c in configs:
        built = c.build(work_dir)
        out.extend(built if isinstance(built, (list, tuple)) else [built])
    return out


@dataclass
class ConcatenatedTokenSourceConfig(TokenSourceConfig):
    sources: List[Any]
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[TokenSource]:
        return [ConcatenatedTokenSource(*_build_all(self.sources, work_dir), work_dir=work_dir, label=self.label)]


@dataclass
class ConcatenatedDocumentSourceConfig(DocumentSourceConfig):
    sources: List[Any]
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[DocumentSource]:
        return [ConcatenatedDocumentSource(*_build_all(self.sources, work_dir), work_dir=work_dir, label=self.label)]


@dataclass
class SplitTokenSourceConfig(TokenSourceConfig):
    source: Any
    ratio: float
    idx: int  # 0: the first part, 1: the second

    def __post_init__(self):
        if not 0 < self.ratio < 1:
            raise ValueError("'ratio' must be strictly between 0 and 1")
        if self.idx not in (0, 1):
            raise ValueError("'idx' must be 0 or 1")

    def build(self, work_dir: PathOrStr) -> List[TokenSource]:
        # several built sources are split as one: the cut falls at ``ratio`` of their total
        # (src/olmo_core/data/composable/token_source.py:447-462)
        sources = _build_all([self.source], work_dir)
        source = sources[0] if len(sources) == 1 else ConcatenatedTokenSource(*sources, work_dir=work_dir)
        return [source.split(self.ratio)[self.idx]]


def _resolve_max_tokens(sources, max_tokens: Optional[int], factor: Optional[float]) -> int:
    if (max_tokens is None) == (factor is None):
        raise ValueError("exactly one of 'max_tokens' and 'factor' is required")
    return max_tokens if max_tokens is not None else int(factor * sum(s.num_tokens for s in sources))  # type: ignore[operator]


ConcatenatedTokenSource.Config = ConcatenatedTokenSourceConfig  # type: ignore[attr-defined]
ConcatenatedDocumentSource.Config = ConcatenatedDocumentSourceConfig  # type: ignore[attr-defined]
