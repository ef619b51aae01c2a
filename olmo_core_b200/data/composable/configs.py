"""
Serializable configs for token and instance sources. Each source class gets its config attached as ``<Source>.Config``
(e.g. ``ConcatAndChunkInstanceSource.Config``, ``MixingInstanceSource.Spec.Config``), mirroring the class attributes of
src/olmo_core/data/composable/{token_source,instance_source,*_source}.py. Token-source configs ``build(work_dir)`` into a
LIST of sources (a glob may expand into many); instance-source configs build into one source.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

from ...aliases import PathOrStr
from ...config import Config
from ..tokenizer import TokenizerConfig
from ..types import LongDocStrategy
from .instance_source import (
    ConcatAndChunkInstanceSource,
    ConcatenatedInstanceSource,
    InstanceSource,
    MixingInstanceSource,
    MixingInstanceSourceSpec,
    PackingInstanceSource,
    RandomInstanceSource,
    SamplingInstanceSource,
    SlicedInstanceSource,
)
from .config_base import DocumentSourceConfig, TokenSourceConfig
from .numpy_document_source import NumpyDocumentSourceConfig, NumpyDocumentSourceMixConfig
from .token_source import (
    ConcatenatedDocumentSource,
    ConcatenatedTokenSource,
    DocumentSource,
    MixingDocumentSource,
    MixingDocumentSourceSpec,
    MixingTokenSource,
    MixingTokenSourceSpec,
    SamplingDocumentSource,
    SamplingTokenSource,
    SlicedTokenSource,
    TokenSource,
)
from .utils import SEED_NOT_SET, resolve_seed

__all__ = [
    "TokenSourceConfig", "DocumentSourceConfig", "ConcatenatedTokenSourceConfig", "ConcatenatedDocumentSourceConfig",
    "SplitTokenSourceConfig", "SamplingTokenSourceConfig", "SamplingDocumentSourceConfig", "MixingTokenSourceConfig",
    "MixingTokenSourceSpecConfig", "MixingDocumentSourceConfig", "MixingDocumentSourceSpecConfig",
    "InstanceSourceConfig", "ConcatAndChunkInstanceSourceConfig", "PackingInstanceSourceConfig",
    "RandomInstanceSourceConfig", "ConcatenatedInstanceSourceConfig", "SplitInstanceSourceConfig",
    "SamplingInstanceSourceConfig", "MixingInstanceSourceConfig", "MixingInstanceSourceSpecConfig",
]


def _default_seed() -> int:
    return resolve_seed(SEED_NOT_SET)


def _build_all(configs: List[Any], work_dir: PathOrStr) -> List[Any]:
    out: List[Any] = []
    for c in configs:
        built = c.build(work_dir)
        out.extend(built if isinstance(built, (list, tuple)) else [built])
    return out


# --------------------------------------------------------------------------------------------------- token sources
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


@dataclass
class SamplingTokenSourceConfig(TokenSourceConfig):
    sources: List[Any]
    max_tokens: Optional[int] = None
    factor: Optional[float] = None
    seed: Optional[int] = field(default_factory=_default_seed)
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[TokenSource]:
        built = _build_all(self.sources, work_dir)
        return [SamplingTokenSource(*built, max_tokens=_resolve_max_tokens(built, self.max_tokens, self.factor),
                                    seed=self.seed, work_dir=work_dir, label=self.label)]


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


@dataclass
class MixingTokenSourceSpecConfig(Config):
    source: Any
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> MixingTokenSourceSpec:
        built = _build_all([self.source], work_dir)
        source = built[0] if len(built) == 1 else ConcatenatedTokenSource(*built, work_dir=work_dir, label=self.label)
        return MixingTokenSourceSpec(source=source, ratio=self.ratio, max_repetition_factor=self.max_repetition_factor,
                                     label=self.label)


@dataclass
class MixingDocumentSourceSpecConfig(MixingTokenSourceSpecConfig):
    def build(self, work_dir: PathOrStr) -> MixingDocumentSourceSpec:  # type: ignore[override]
        built = _build_all([self.source], work_dir)
        source = built[0] if len(built) == 1 else ConcatenatedDocumentSource(*built, work_dir=work_dir, label=self.label)
        return MixingDocumentSourceSpec(source=source, ratio=self.ratio, max_repetition_factor=self.max_repetition_factor,
                                        label=self.label)


@dataclass
class MixingTokenSourceConfig(TokenSourceConfig):
    source_specs: List[MixingTokenSourceSpecConfig]
    seed: Optional[int] = field(default_factory=_default_seed)
    num_tokens: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[TokenSource]:
        return [MixingTokenSource(*[s.build(work_dir) for s in self.source_specs], work_dir=work_dir, seed=self.seed,
                                  num_tokens=self.num_tokens, label=self.label)]


@dataclass
class MixingDocumentSourceConfig(DocumentSourceConfig):
    source_specs: List[MixingDocumentSourceSpecConfig]
    seed: Optional[int] = field(default_factory=_default_seed)
    num_tokens: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[DocumentSource]:
        return [MixingDocumentSource(*[s.build(work_dir) for s in self.source_specs], work_dir=work_dir, seed=self.seed,
                                     num_tokens=self.num_tokens, label=self.label)]


# ------------------------------------------------------------------------------------------------ instance sources
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
class ConcatAndChunkInstanceSourceConfig(InstanceSourceConfig):
    sources: List[Any]  # token source configs
    sequence_length: int
    max_sequence_length: Optional[int] = None
    label: Optional[str] = None

    @classmethod
    def from_npy(cls, *npy_paths: str, tokenizer: TokenizerConfig, sequence_length: int,
                 max_sequence_length: Optional[int] = None, dtype=None, source_permutation_seed: Optional[int] = None,
                 source_group_size: int = 1, label_mask_paths: Optional[List[str]] = None,
                 expand_glob: Optional[bool] = None, label: Optional[str] = None) -> "ConcatAndChunkInstanceSourceConfig":
        """Instances cut from one or more tokenized ``.npy`` files."""
        from .numpy_document_source import NumpyDocumentSourceConfig

        return cls(sources=[NumpyDocumentSourceConfig(
            source_paths=list(npy_paths), tokenizer=tokenizer, dtype=dtype,
            source_permutation_seed=resolve_seed(source_permutation_seed), source_group_size=source_group_size,
            label_mask_paths=label_mask_paths, expand_glob=expand_glob)],
            sequence_length=sequence_length, max_sequence_length=max_sequence_length, label=label)

    def build(self, work_dir: PathOrStr) -> ConcatAndChunkInstanceSource:
        return ConcatAndChunkInstanceSource(*_build_all(self.sources, work_dir), sequence_length=self.sequence_length,
                                            max_sequence_length=self.max_sequence_length, work_dir=work_dir,
                                            label=self.label)


@dataclass
class PackingInstanceSourceConfig(InstanceSourceConfig):
    sources: List[Any]  # document source configs
    sequence_length: int
    tokenizer: TokenizerConfig
    max_sequence_length: Optional[int] = None
    long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate
    source_group_size: int = 1
    label: Optional[str] = None

    @classmethod
    def from_npy(cls, *npy_paths: str, tokenizer: TokenizerConfig, sequence_length: int,
                 max_sequence_length: Optional[int] = None, dtype=None, source_permutation_seed: Optional[int] = None,
                 source_group_size: int = 1, label_mask_paths: Optional[List[str]] = None,
                 expand_glob: Optional[bool] = None, label: Optional[str] = None,
                 long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate) -> "PackingInstanceSourceConfig":
        """Whole documents of one or more tokenized ``.npy`` files packed into instances."""
        from .numpy_document_source import NumpyDocumentSourceConfig

        return cls(sources=[NumpyDocumentSourceConfig(
            source_paths=list(npy_paths), tokenizer=tokenizer, dtype=dtype,
            source_permutation_seed=resolve_seed(source_permutation_seed), source_group_size=source_group_size,
            label_mask_paths=label_mask_paths, expand_glob=expand_glob)],
            sequence_length=sequence_length, tokenizer=tokenizer, max_sequence_length=max_sequence_length, label=label,
            long_doc_strategy=long_doc_strategy, source_group_size=source_group_size)

    def build(self, work_dir: PathOrStr) -> PackingInstanceSource:
        return PackingInstanceSource(*_build_all(self.sources, work_dir), sequence_length=self.sequence_length,
                                     max_sequence_length=self.max_sequence_length,
                                     tokenizer=self.tokenizer, long_doc_strategy=self.long_doc_strategy,
                                     source_group_size=self.source_group_size, work_dir=work_dir, label=self.label)


@dataclass
class RandomInstanceSourceConfig(InstanceSourceConfig):
    tokenizer: TokenizerConfig
    sequence_length: int
    avg_document_length: int
    seed: Optional[int] = field(default_factory=_default_seed)
    num_instances: Optional[int] = None
    num_tokens: Optional[int] = None
    max_sequence_length: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> RandomInstanceSource:
        return RandomInstanceSource(tokenizer=self.tokenizer, sequence_length=self.sequence_length,
                                    avg_document_length=self.avg_document_length, seed=self.seed,
                                    num_instances=self.num_instances, num_tokens=self.num_tokens,
                                    max_sequence_length=self.max_sequence_length, label=self.label, work_dir=work_dir)


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


@dataclass
class MixingInstanceSourceSpecConfig(Config):
    source: InstanceSourceConfig
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> MixingInstanceSourceSpec:
        return MixingInstanceSourceSpec(source=self.source.build(work_dir), ratio=self.ratio,
                                        max_repetition_factor=self.max_repetition_factor, label=self.label)


@dataclass
class MixingInstanceSourceConfig(InstanceSourceConfig):
    source_specs: List[MixingInstanceSourceSpecConfig]
    seed: Optional[int] = field(default_factory=_default_seed)
    num_tokens: Optional[int] = None
    num_instances: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> MixingInstanceSource:
        return MixingInstanceSource(*[s.build(work_dir) for s in self.source_specs], work_dir=work_dir, seed=self.seed,
                                    num_tokens=self.num_tokens, num_instances=self.num_instances, label=self.label)


# the token-source configs of numpy files are document-source configs
for _cls in (NumpyDocumentSourceConfig, NumpyDocumentSourceMixConfig):
    for _name in ("__add__", "__mul__", "sample", "resize", "split"):
        setattr(_cls, _name, getattr(TokenSourceConfig, _name))
    for _name in ("sample_by_docs", "resize_by_docs"):
        setattr(_cls, _name, getattr(DocumentSourceConfig, _name))

ConcatenatedTokenSource.Config = ConcatenatedTokenSourceConfig  # type: ignore[attr-defined]
ConcatenatedDocumentSource.Config = ConcatenatedDocumentSourceConfig  # type: ignore[attr-defined]
SlicedTokenSource.Config = SplitTokenSourceConfig  # type: ignore[attr-defined]
SamplingTokenSource.Config = SamplingTokenSourceConfig  # type: ignore[attr-defined]
SamplingDocumentSource.Config = SamplingDocumentSourceConfig  # type: ignore[attr-defined]
MixingTokenSource.Config = MixingTokenSourceConfig  # type: ignore[attr-defined]
MixingTokenSourceSpec.Config = MixingTokenSourceSpecConfig  # type: ignore[attr-defined]
MixingDocumentSource.Config = MixingDocumentSourceConfig  # type: ignore[attr-defined]
MixingDocumentSourceSpec.Config = MixingDocumentSourceSpecConfig  # type: ignore[attr-defined]
ConcatAndChunkInstanceSource.Config = ConcatAndChunkInstanceSourceConfig  # type: ignore[attr-defined]
PackingInstanceSource.Config = PackingInstanceSourceConfig  # type: ignore[attr-defined]
RandomInstanceSource.Config = RandomInstanceSourceConfig  # type: ignore[attr-defined]
ConcatenatedInstanceSource.Config = ConcatenatedInstanceSourceConfig  # type: ignore[attr-defined]
SlicedInstanceSource.Config = SplitInstanceSourceConfig  # type: ignore[attr-defined]
SamplingInstanceSource.Config = SamplingInstanceSourceConfig  # type: ignore[attr-defined]
MixingInstanceSource.Config = MixingInstanceSourceConfig  # type: ignore[attr-defined]
MixingInstanceSourceSpec.Config = MixingInstanceSourceSpecConfig  # type: ignore[attr-defined]
