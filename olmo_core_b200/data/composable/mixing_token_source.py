"""Token sources mixed at given ratios (src/olmo_core/data/composable/mixing_token_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional

from ...aliases import PathOrStr
from ...config import Config
from .sampling_token_source import SamplingTokenSource
from .token_source import (
    ConcatenatedTokenSource,
    TokenSource,
    TokenSourceConfig,
    _Spliced,
    _build_all,
    _default_seed,
    _whole,
)
from .utils import SEED_NOT_SET, calculate_sample_sizes, resolve_seed

__all__ = ["MixingTokenSource", "MixingTokenSourceSpec", "MixingTokenSourceConfig", "MixingTokenSourceSpecConfig"]


@dataclass
class MixingTokenSourceSpec:
    source: TokenSource
    ratio: float
    max_repetition_factor: float = 1.0
    label: Optional[str] = None


class MixingTokenSource(ConcatenatedTokenSource):
    """Sources combined at given ratios: each is sampled to the size the ratios call for, then concatenated."""

    DISPLAY_ICON = ""
    Spec = MixingTokenSourceSpec
    _sampler: Any = SamplingTokenSource  # how each source is brought to its share

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
            sampled.append(self._sampler(spec.source, max_tokens=int(size), seed=child_seed, work_dir=work_dir, label=labels[i]))
        self.sampled_sources = tuple(sampled)
        _Spliced.__init__(self, sampled, _whole(sampled), work_dir=work_dir, label=label)

    @property
    def seed(self) -> Optional[int]:
        return self._seed


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
class MixingTokenSourceConfig(TokenSourceConfig):
    source_specs: List[MixingTokenSourceSpecConfig]
    seed: Optional[int] = field(default_factory=_default_seed)
    num_tokens: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> List[TokenSource]:
        return [MixingTokenSource(*[s.build(work_dir) for s in self.source_specs], work_dir=work_dir, seed=self.seed,
                                  num_tokens=self.num_tokens, label=self.label)]


MixingTokenSource.Config = MixingTokenSourceConfig  # type: ignore[attr-defined]
MixingTokenSourceSpec.Config = MixingTokenSourceSpecConfig  # type: ignore[attr-defined]
