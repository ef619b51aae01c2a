"""Instances cut consecutively from token sources (src/olmo_core/data/composable/concat_and_chunk_instance_source.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import numpy as np

from ...aliases import PathOrStr
from ..tokenizer import TokenizerConfig
from .instance_source import Instance, InstanceSource, InstanceSourceConfig
from .token_source import TokenSource, _build_all
from .utils import as_ndarray, resolve_seed

__all__ = ["ConcatAndChunkInstanceSource", "ConcatAndChunkInstanceSourceConfig"]


class ConcatAndChunkInstanceSource(InstanceSource):
    """Each token source is cut into consecutive instances; document boundaries are ignored."""

    DISPLAY_ICON = ""

    def __init__(self, *sources: TokenSource, sequence_length: int, max_sequence_length: Optional[int] = None,
                 work_dir: PathOrStr, label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, max_sequence_length=max_sequence_length,
                         label=label)
        self._sources = tuple(sources)
        per_source = [s.num_tokens // self.max_sequence_length * (self.max_sequence_length // sequence_length)
                      for s in sources]
        self._ends = np.cumsum(per_source)

    @property
    def sources(self) -> Tuple[TokenSource, ...]:
        return self._sources

    def children(self):
        return self._sources

    @property
    def fingerprint(self) -> str:
        return self._hash(*[s.fingerprint for s in self._sources], self.sequence_length, self.max_sequence_length)

    def __len__(self) -> int:
        return int(self._ends[-1])

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        k = int(np.searchsorted(self._ends, idx, side="right"))
        local = idx - (int(self._ends[k - 1]) if k else 0)
        rng = self._sources[k].get_token_range(local * self.sequence_length, (local + 1) * self.sequence_length)
        out: Instance = {"input_ids": as_ndarray(rng["input_ids"])}
        if "label_mask" in rng:
            out["label_mask"] = as_ndarray(rng["label_mask"])
        return out


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


ConcatAndChunkInstanceSource.Config = ConcatAndChunkInstanceSourceConfig  # type: ignore[attr-defined]
