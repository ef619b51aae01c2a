"""
Interleaved documents (behaviour of src/olmo_core/data/numpy_dataset.py:1343-1620): ``docs_per_instance`` documents,
drawn by a seeded permutation, are stripped of special tokens, cut into ``chunks_per_doc`` chunks each and woven
together chunk by chunk (``a0 b0 a1 b1 ...``) into one instance -- long-context training data made of unrelated
documents whose pieces are far apart. Documents of ``interleaving_exempt_paths`` are served as they are, first.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ...aliases import PathOrStr
from ...distributed.utils import barrier
from ...exceptions import OLMoConfigurationError
from ..utils import get_rng, write_array_to_disk
from .base import locate
from .fsl import NumpyPaddedFSLDataset, _mmap

log = logging.getLogger(__name__)

__all__ = ["NumpyInterleavedFSLDataset"]


class NumpyInterleavedFSLDataset(NumpyPaddedFSLDataset):
    def __init__(self, *paths: PathOrStr, sequence_length: int, seed: int, docs_per_instance: int, chunks_per_doc: int,
                 interleaving_exempt_paths: Optional[Sequence[PathOrStr]] = None, **kwargs):
        if sequence_length % docs_per_instance != 0:
            raise OLMoConfigurationError("'sequence_length' must be a multiple of 'docs_per_instance'")
        if sequence_length % chunks_per_doc != 0:
            raise OLMoConfigurationError("'sequence_length' must be a multiple of 'chunks_per_doc'")
        kwargs.pop("generate_doc_lengths", None)
        super().__init__(*paths, sequence_length=sequence_length, **kwargs)
        self._docs_per_instance = docs_per_instance
        self._chunks_per_doc = chunks_per_doc
        self._seed = seed
        self._interleaving_exempt_paths = list(interleaving_exempt_paths) if interleaving_exempt_paths else None
        self._order: Optional[np.ndarray] = None
        self._exempt: Optional[np.ndarray] = None

    @property
    def fingerprint_fields(self) -> Tuple[str, ...]:
        return ("vocab_size", "pad_token_id", "eos_token_id", "dtype", "_docs_per_instance", "_seed",
                "_interleaving_exempt_paths", "max_target_sequence_length", "bos_token_id", "sequence_length")

    def _get_instance_indices_path(self, source_path: PathOrStr) -> Path:
        return self._cache_path("instance-indices", source_path, seq=self.sequence_length, docs=self._docs_per_instance,
                                dt=np.dtype(self.indices_dtype).name)

    def _order_paths(self) -> Tuple[Path, Path]:
        root = self.work_dir / f"dataset-{self.fingerprint}"
        return root / "interleavable-docs-indices.npy", root / "interleaving-exempt-docs-indices.npy"

    def prepare(self) -> None:
        if self.fs_local_rank == 0:
            self._write_instance_indices()
            self._write_order()
        barrier()
        len(self)

    def _write_order(self) -> None:
        order_path, exempt_path = self._order_paths()
        if order_path.is_file() and (self._interleaving_exempt_paths is None or exempt_path.is_file()):
            return
        n_docs = self.offsets[-1][1]
        exempt_mask = np.zeros(n_docs, dtype=bool)
        if self._interleaving_exempt_paths:
            for i, (start, end) in enumerate(self.offsets):
                if self.paths[i] in self._interleaving_exempt_paths:
                    exempt_mask[start:end] = True
            write_array_to_disk(np.nonzero(exempt_mask)[0].astype(self.indices_dtype), exempt_path)
        free = np.nonzero(~exempt_mask)[0]
        write_array_to_disk(get_rng(self._seed).permutation(free).astype(self.indices_dtype), order_path)

    def _load_order(self) -> Tuple[np.ndarray, np.ndarray]:
        if self._order is None:
            order_path, exempt_path = self._order_paths()
            self._order = _mmap(order_path, self.indices_dtype)
            self._exempt = _mmap(exempt_path, self.indices_dtype) if exempt_path.is_file() else np.zeros(0, dtype=self.indices_dtype)
        assert self._exempt is not None
        return self._order, self._exempt

    def __len__(self) -> int:
        order, exempt = self._load_order()
        return len(order) // self._docs_per_instance + len(exempt)

    def _source_of(self, index: int) -> Tuple[int, int]:
        # indices handed to the padded base class address DOCUMENTS, of which there are more than instances
        offsets = self.offsets
        if self._starts is None:
            self._starts = [o[0] for o in offsets]
        return locate(offsets, self._starts, int(index), offsets[-1][1])

    def _weave(self, parts: List[torch.Tensor]) -> torch.Tensor:
        chunks = [p.tensor_split(self._chunks_per_doc) for p in parts]
        return torch.cat([doc_chunks[i] for i in range(self._chunks_per_doc) for doc_chunks in chunks])

    def __getitem__(self, index: int) -> Dict[str, Any]:
        order, exempt = self._load_order()
        pos = int(index) if index >= 0 else len(self) + int(index)
        if pos < len(exempt):
            return super().__getitem__(int(exempt[pos]))
        pos -= len(exempt)
        k, L = self._docs_per_instance, self.sequence_length
        share = L // k
        docs = [super(NumpyInterleavedFSLDataset, self).__getitem__(int(d)) for d in order[pos * k: (pos + 1) * k]]
        if any(d.keys() != docs[0].keys() for d in docs):
            raise RuntimeError("cannot interleave documents that carry different fields")
        ids_parts, mask_parts = [], []
        for d in docs:
            ids, mask = d["input_ids"][:share], d["label_mask"][:share]
            special = (ids == self.pad_token_id) | (ids == self.eos_token_id)
            if self.bos_token_id is not None:
                special |= ids == self.bos_token_id
            ids_parts.append(ids[~special])
            mask_parts.append(mask[~special])
        ids, mask = self._weave(ids_parts), self._weave(mask_parts)
        # re-frame the woven sequence as one document, then pad
        if self.bos_token_id is not None and len(ids) < L:
            ids = torch.cat([ids.new_tensor([self.bos_token_id]), ids])
            mask = torch.cat([mask.new_tensor([True]), mask])
        if len(ids) < L:
            ids = torch.cat([ids, ids.new_tensor([self.eos_token_id])])
            mask = torch.cat([mask, mask.new_tensor([True])])
        item = self._pad({"input_ids": ids, "label_mask": mask})
        if "instance_mask" in docs[0]:
            item["instance_mask"] = all(d["instance_mask"] for d in docs)
        if "metadata" in docs[0]:
            if any(d["metadata"] != docs[0]["metadata"] for d in docs):
                raise RuntimeError("cannot interleave documents with different metadata")
            item["metadata"] = docs[0]["metadata"]
        return item
