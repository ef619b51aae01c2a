"""
Bases of the token / document source configs (src/olmo_core/data/composable/token_source.py:109-203,
document-source counterpart at 352-420). They live apart from the concrete configs so that source modules can derive
their own configs from them; the sampling / splitting configs they return are imported when first used.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, List, Optional, Tuple

from ...aliases import PathOrStr
from ...config import Config
from .utils import SEED_NOT_SET, resolve_seed

if TYPE_CHECKING:
    from .configs import (
        ConcatenatedTokenSourceConfig,
        SamplingDocumentSourceConfig,
        SamplingTokenSourceConfig,
        SplitTokenSourceConfig,
    )
    from .token_source import DocumentSource, TokenSource

__all__ = ["TokenSourceConfig", "DocumentSourceConfig"]


@dataclass
class TokenSourceConfig(Config):
    def build(self, work_dir: PathOrStr) -> List["TokenSource"]:
        raise NotImplementedError

    def __add__(self, other: "TokenSourceConfig") -> "TokenSourceConfig":
        """Concatenation; two document sources give a document source."""
        from .configs import ConcatenatedDocumentSourceConfig, ConcatenatedTokenSourceConfig

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
        from .configs import SamplingTokenSourceConfig

        return SamplingTokenSourceConfig(sources=[self], max_tokens=max_tokens, factor=factor, seed=resolve_seed(seed))

    def resize(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingTokenSourceConfig":
        return self.sample(factor=factor, seed=seed)

    def split(self, ratio: float) -> Tuple["SplitTokenSourceConfig", "SplitTokenSourceConfig"]:
        from .configs import SplitTokenSourceConfig

        return (SplitTokenSourceConfig(source=self, ratio=ratio, idx=0), SplitTokenSourceConfig(source=self, ratio=ratio, idx=1))


@dataclass
class DocumentSourceConfig(TokenSourceConfig):
    def build(self, work_dir: PathOrStr) -> List["DocumentSource"]:  # type: ignore[override]
        raise NotImplementedError

    def sample_by_docs(self, *, max_tokens: Optional[int] = None, factor: Optional[float] = None,
                       seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSourceConfig":
        from .configs import SamplingDocumentSourceConfig

        return SamplingDocumentSourceConfig(sources=[self], max_tokens=max_tokens, factor=factor, seed=resolve_seed(seed))

    def resize_by_docs(self, factor: float, seed: Optional[int] = SEED_NOT_SET) -> "SamplingDocumentSourceConfig":
        return self.sample_by_docs(factor=factor, seed=seed)
