"""Whole documents packed into instances (src/olmo_core/data/composable/packing_instance_source.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import numpy as np

from ...aliases import PathOrStr
from ..tokenizer import TokenizerConfig
from ..types import LongDocStrategy
from ..utils import InstancePacker
from .instance_source import Instance, InstanceSource, InstanceSourceConfig
from .token_source import DocumentSource, _build_all
from .utils import as_ndarray, resolve_seed

__all__ = ["PackingInstanceSource", "PackingInstanceSourceConfig"]


class PackingInstanceSource(InstanceSource):
    """
    Whole documents packed into instances with best-fit-decreasing bin packing; the tail of every instance is padding
    (masked out of the loss). Documents longer than an instance are truncated or split, per ``long_doc_strategy``.
    Sources are packed in groups of ``source_group_size`` so that instances rarely mix distant sources.
    """

    DISPLAY_ICON = ""

    def __init__(self, *sources: DocumentSource, sequence_length: int, work_dir: PathOrStr, tokenizer=None,
                 pad_token_id: Optional[int] = None, max_sequence_length: Optional[int] = None,
                 long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate, source_group_size: int = 1,
                 label: Optional[str] = None):
        if not sources:
            raise ValueError("At least one source must be provided.")
        if tokenizer is not None:
            pad_token_id = tokenizer.pad_token_id
        if pad_token_id is None:
            raise ValueError("a tokenizer config (or 'pad_token_id') is required")
        self._tokenizer = tokenizer
        if max_sequence_length not in (None, sequence_length):
            raise ValueError("packed instances cannot be re-cut: 'max_sequence_length' must equal 'sequence_length'")
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, label=label)
        self._sources = tuple(sources)
        self._pad = pad_token_id
        self._strategy = LongDocStrategy(long_doc_strategy)
        self._group_size = source_group_size
        # instance -> rows of the document table; document table rows are (source index, start, end)
        self._docs = np.empty((0, 3), dtype=np.int64)
        self._instance_docs: List[List[int]] = []
        for g in range(0, len(sources), source_group_size):
            rows = []
            for i in range(g, min(g + source_group_size, len(sources))):
                for s, e in sources[i].get_document_offsets():
                    rows.extend(self._fit(i, s, e))
            table = np.array(rows, dtype=np.int64).reshape(-1, 3)
            packer = InstancePacker(sequence_length)
            instances, _, _ = packer.pack_documents(table[:, 1:])
            table = table[packer.last_order]  # the instances refer to the documents longest first
            base = len(self._docs)
            self._instance_docs.extend([[base + d for d in inst] for inst in instances])
            self._docs = np.concatenate([self._docs, table], axis=0)

    def _fit(self, source: int, start: int, end: int) -> List[Tuple[int, int, int]]:
        L = self.sequence_length
        if end - start <= L:
            return [(source, start, end)]
        if self._strategy == LongDocStrategy.truncate:
            return [(source, start, start + L)]
        return [(source, s, min(end, s + L)) for s in range(start, end, L)]

    def children(self):
        return self._sources

    @property
    def sources(self) -> Tuple[DocumentSource, ...]:
        return self._sources

    @property
    def source_groups(self) -> Tuple[Tuple[DocumentSource, ...], ...]:
        return tuple(self._sources[g:g + self._group_size] for g in range(0, len(self._sources), self._group_size))

    @property
    def source_group_size(self) -> int:
        return self._group_size

    @property
    def long_doc_strategy(self) -> LongDocStrategy:
        return self._strategy

    @property
    def pad_token_id(self) -> int:
        return self._pad

    @property
    def num_instances(self) -> int:
        return len(self._instance_docs)

    @property
    def fingerprint(self) -> str:
        return self._hash(*[s.fingerprint for s in self._sources], self.sequence_length, self._pad, self._strategy,
                          self._group_size)

    def __len__(self) -> int:
        return len(self._instance_docs)

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        ids = np.full(self.sequence_length, self._pad, dtype=np.int64)
        mask = np.zeros(self.sequence_length, dtype=bool)
        pos = 0
        for d in self._instance_docs[idx]:
            src, s, e = (int(v) for v in self._docs[d])
            rng = self._sources[src].get_token_range(s, e)
            n = e - s
            ids[pos:pos + n] = as_ndarray(rng["input_ids"])
            mask[pos:pos + n] = as_ndarray(rng["label_mask"]) if "label_mask" in rng else True
            pos += n
        return {"input_ids": ids, "label_mask": mask}


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


PackingInstanceSource.Config = PackingInstanceSourceConfig  # type: ignore[attr-defined]
