"""Instance sources mixed at given ratios (src/olmo_core/data/composable/mixing_instance_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ...aliases import PathOrStr
from ...config import Config
from ...exceptions import OLMoConfigurationError
from .instance_source import InstanceSource, InstanceSourceConfig, _all_of, _Indexed
from .sampling_instance_source import SamplingInstanceSource
from .token_source import _default_seed
from .utils import SEED_NOT_SET, calculate_sample_sizes, resolve_seed

__all__ = ["MixingInstanceSource", "MixingInstanceSourceSpec", "MixingInstanceSourceConfig",
           "MixingInstanceSourceSpecConfig"]


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


MixingInstanceSource.Config = MixingInstanceSourceConfig  # type: ignore[attr-defined]
MixingInstanceSourceSpec.Config = MixingInstanceSourceSpecConfig  # type: ignore[attr-defined]
