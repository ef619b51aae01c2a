"""Token-level sampling of token sources (src/olmo_core/data/composable/sampling_token_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence

from ...aliases import PathOrStr
from ..utils import get_rng
from .sliced_token_source import SlicedTokenSource
from .token_source import TokenSource, TokenSourceConfig, _Spliced, _build_all, _default_seed, _resolve_max_tokens, _whole
from .utils import SEED_NOT_SET, resolve_seed

__all__ = ["SamplingTokenSource", "SamplingTokenSourceConfig"]


def _unwind(sources: Sequence[TokenSource]) -> List[TokenSource]:
    """
    Replace mixes by their per-source samples and samples by the pieces they are made of, breadth first (the order of
    src/olmo_core/data/composable/sampling_token_source.py:103-120), so that re-sampling keeps THEIR proportions.
    """
    from collections import deque

    from .mixing_token_source import MixingTokenSource

    out: List[TokenSource] = []
    frontier = deque(sources)
    while frontier:
        s = frontier.popleft()
        if isinstance(s, MixingTokenSource):  # document mixes derive from it
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


SamplingTokenSource.Config = SamplingTokenSourceConfig  # type: ignore[attr-defined]
