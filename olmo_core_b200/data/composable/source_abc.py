"""Common base of token and instance sources (role of src/olmo_core/data/composable/source_abc.py:11-93)."""

from __future__ import annotations

import hashlib
from abc import ABCMeta, abstractmethod
from pathlib import Path
from typing import Iterable, Optional

from ...aliases import PathOrStr
from ...distributed.utils import get_fs_local_rank, get_rank
from ...io import is_url, normalize_path

__all__ = ["SourceABC"]


class SourceABC(metaclass=ABCMeta):
    """
    A node in a tree of data sources. Every node has a content ``fingerprint`` (used to name cache files, so two
    differently composed sources never share a cache entry), a size in tokens and its child sources.
    """

    DISPLAY_ICON = ""

    def __init__(self, *, work_dir: PathOrStr, label: Optional[str] = None):
        if is_url(work_dir):
            raise ValueError(f"'work_dir' must be a local directory, got '{work_dir}'")
        self._common_work_dir = Path(normalize_path(work_dir))
        self._label = label
        self._fs_local_rank = get_fs_local_rank()
        self._rank = get_rank()

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.fingerprint[:7]})"

    @property
    def common_work_dir(self) -> Path:
        """The directory shared by all sources of a tree."""
        return self._common_work_dir

    @property
    def work_dir(self) -> Path:
        """This class's own sub-directory for cache files."""
        return self._common_work_dir / type(self).__name__

    @property
    def fs_local_rank(self) -> int:
        return self._fs_local_rank

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def label(self) -> Optional[str]:
        return self._label

    @property
    @abstractmethod
    def fingerprint(self) -> str:
        raise NotImplementedError

    @property
    @abstractmethod
    def num_tokens(self) -> int:
        raise NotImplementedError

    @abstractmethod
    def children(self) -> Iterable["SourceABC"]:
        raise NotImplementedError

    @property
    def is_leaf(self) -> bool:
        return not list(self.children())

    def _hash(self, *parts) -> str:
        """Fingerprint from the class name and the given parts (child fingerprints, parameters)."""
        h = hashlib.sha256(f"class={type(self).__name__},".encode())
        for part in parts:
            h.update(f"{part},".encode())
        return h.hexdigest()
