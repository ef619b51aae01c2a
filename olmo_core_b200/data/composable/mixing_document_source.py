"""Document sources mixed at given ratios, sampled by whole documents
(src/olmo_core/data/composable/mixing_document_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Tuple

from ...aliases import PathOrStr
from .mixing_token_source import MixingTokenSource, MixingTokenSourceSpecConfig
from .sampling_document_source import SamplingDocumentSource
from .token_source import ConcatenatedDocumentSource, DocumentSource, DocumentSourceConfig, _build_all, _default_seed

__all__ = ["MixingDocumentSource", "MixingDocumentSourceSpec", "MixingDocumentSourceConfig",
           "MixingDocumentSourceSpecConfig"]


@dataclass
class MixingDocumentSourceSpec:
    source: DocumentSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None


class MixingDocumentSource(MixingTokenSource, DocumentSource):
    Spec = MixingDocumentSourceSpec
    _sampler = SamplingDocumentSource

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        base = 0
        for child in self.sampled_sources:
            for s, e in child.get_document_offsets():
                yield base + s, base + e
            base += child.num_tokens


@dataclass
class MixingDocumentSourceSpecConfig(MixingTokenSourceSpecConfig):
    def build(self, work_dir: PathOrStr) -> MixingDocumentSourceSpec:  # type: ignore[override]
        built = _build_all([self.source], work_dir)
        source = built[0] if len(built) == 1 else ConcatenatedDocumentSource(*built, work_dir=work_dir, label=self.label)
        return MixingDocumentSourceSpec(source=source, ratio=self.ratio, max_repetition_factor=self.max_repetition_factor,
                                        label=self.label)


@dataclass
class MixingDocumentSourceConfig(DocumentSourceConfig):
    source_specs: List[MixingDocumentSourceSpecConfig]
    seed: Optional[int] = field(default_factory=_default_seed)
    num_tokens: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[DocumentSource]:
        return [MixingDocumentSource(*[s.build(work_dir) for s in self.source_specs], work_dir=work_dir, seed=self.seed,
                                     num_tokens=self.num_tokens, label=self.label)]


MixingDocumentSource.Config = MixingDocumentSourceConfig  # type: ignore[attr-defined]
MixingDocumentSourceSpec.Config = MixingDocumentSourceSpecConfig  # type: ignore[attr-defined]
