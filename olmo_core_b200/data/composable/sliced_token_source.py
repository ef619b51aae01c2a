"""A contiguous slice of a token source (src/olmo_core/data/composable/sliced_token_source.py)."""

from __future__ import annotations

from typing import Optional

import numpy as np

from ...aliases import PathOrStr
from .token_source import SplitTokenSourceConfig, TokenSource, _Spliced

__all__ = ["SlicedTokenSource"]


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


SlicedTokenSource.Config = SplitTokenSourceConfig  # type: ignore[attr-defined]
