"""Document-level sampling of document sources (src/olmo_core/data/composable/sampling_document_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable, List, Optional, Tuple

import numpy as np

from ...aliases import PathOrStr
from ..utils import get_rng
from .token_source import (
    ConcatenatedDocumentSource,
    DocumentSource,
    DocumentSourceConfig,
    _Spliced,
    _build_all,
    _default_seed,
    _resolve_max_tokens,
)
from .utils import SEED_NOT_SET, resolve_seed

__all__ = ["SamplingDocumentSource", "SamplingDocumentSourceConfig"]


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
class SamplingDocumentSourceConfig(DocumentSourceConfig):
    sources: List[Any]
    max_tokens: Optional[int] = None
    factor: Optional[float] = None
    seed: Optional[int] = field(default_factory=_default_seed)
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[DocumentSource]:
        built = _build_all(self.sources, work_dir)
        return [SamplingDocumentSource(*built, max_tokens=_resolve_max_tokens(built, self.max_tokens, self.factor),
                                       seed=self.seed, work_dir=work_dir, label=self.label)]


SamplingDocumentSource.Config = SamplingDocumentSourceConfig  # type: ignore[attr-defined]
