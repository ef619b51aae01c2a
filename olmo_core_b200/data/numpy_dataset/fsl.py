"""
Fixed-sequence-length datasets over token ``.npy`` files
(behaviour of src/olmo_core/data/numpy_dataset.py:451-1620):

* :class:`NumpyFSLDataset` -- every file is cut into consecutive ``sequence_length`` windows ("concat and chunk");
* :class:`NumpyFSLDatasetMixture` -- the same, using only the first ``path_offset_index[(path, i)]`` tokens of each file;
* :class:`NumpyPaddedFSLDataset` -- one document per instance, truncated to ``sequence_length`` and padded;
* :class:`NumpyPackedFSLDataset` -- whole documents bin-packed (best fit decreasing) into instances, padded;

Derived index tables live in the work directory as raw little-endian arrays and are memory-mapped on first use.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ...aliases import PathOrStr
from ...distributed.utils import barrier
from ...exceptions import OLMoConfigurationError, OLMoEnvironmentError
from ...io import get_file_size
from ..types import LongDocStrategy, NumpyUIntTypes
from ..utils import (
    InstancePacker,
    chunked,
    get_document_lengths,
    get_rng,
    iter_document_indices,
    load_array_slice_into_tensor,
    segment_documents_into_instances,
    write_array_to_disk,
)
from .base import InstanceFilterConfig, NumpyFSLDatasetBase, locate

log = logging.getLogger(__name__)

__all__ = ["NumpyFSLDataset", "NumpyFSLDatasetMixture", "NumpyPaddedFSLDataset", "NumpyPackedFSLDataset"]


def _cumulative(counts: Sequence[int]) -> Tuple[Tuple[int, int], ...]:
    out, start = [], 0
    for n in counts:
        out.append((start, start + n))
        start += n
    return tuple(out)


def _mmap(path: Path, dtype) -> np.ndarray:
    return np.memmap(path, mode="r", dtype=dtype)


class NumpyFSLDataset(NumpyFSLDatasetBase):
    """
    With ``max_target_sequence_length`` (a multiple of ``sequence_length``) only as many tokens of each file are used
    as the larger length would use, so that runs at different sequence lengths see the same tokens in the same order.
    """

    def __init__(self, *paths: PathOrStr, sequence_length: int, max_target_sequence_length: Optional[int] = None, **kwargs):
        super().__init__(*paths, sequence_length=sequence_length, **kwargs)
        if max_target_sequence_length is not None and (
            max_target_sequence_length < sequence_length or max_target_sequence_length % sequence_length != 0
        ):
            raise OLMoConfigurationError(
                f"'max_target_sequence_length'({max_target_sequence_length}) should be a multiple of "
                f"'sequence_length'({sequence_length})"
            )
        self._max_target_sequence_length = max_target_sequence_length
        self._array_offsets: Optional[Tuple[Tuple[int, int], ...]] = None
        self._starts: Optional[List[int]] = None
        self._num_instances: Optional[int] = None

    @property
    def fingerprint_fields(self) -> Tuple[str, ...]:
        return ("vocab_size", "pad_token_id", "eos_token_id", "dtype", "max_target_sequence_length", "bos_token_id",
                "sequence_length")

    @property
    def num_tokens(self) -> int:
        return len(self) * self.sequence_length

    @property
    def max_target_sequence_length(self) -> Optional[int]:
        return self._max_target_sequence_length

    @property
    def file_sizes(self) -> Tuple[int, ...]:
        return self._sizes_and_offsets[0]

    @property
    def offsets(self) -> Tuple[Tuple[int, int], ...]:
        """``(first, last + 1)`` global instance index of every source file."""
        return self._sizes_and_offsets[1]

    def prepare(self) -> None:
        len(self)

    def __len__(self) -> int:
        if self._num_instances is None:
            self._num_instances = self.offsets[-1][1]
        return self._num_instances

    def _source_of(self, index: int) -> Tuple[int, int]:
        offsets = self.offsets
        if self._starts is None:
            self._starts = [o[0] for o in offsets]
        return locate(offsets, self._starts, int(index), len(self))

    def __getitem__(self, index: int) -> Dict[str, Any]:
        src, local = self._source_of(index)
        input_ids = self._read_chunk_from_array(self.paths[src], local)
        out: Dict[str, Any] = {"input_ids": input_ids}
        if self._label_mask_paths is not None:
            out["label_mask"] = self._read_chunk_from_array(self._label_mask_paths[src], local, dtype=np.bool_)
        if self.instance_filter_config is not None:
            out["instance_mask"] = self._validate_instance(input_ids, self.instance_filter_config)
        if self._include_instance_metadata:
            out["metadata"] = self._instance_metadata(src)
        if self._generate_doc_lengths:
            out["doc_lens"] = get_document_lengths(input_ids, self.eos_token_id, bos_token_id=self.bos_token_id)
        return out

    @property
    def _sizes_and_offsets(self) -> Tuple[Tuple[int, ...], Tuple[Tuple[int, int], ...]]:
        if self._array_offsets is None or self._array_file_sizes is None:
            results = self.map(self._get_file_size_and_length)
            self._array_file_sizes = tuple(size for size, _ in results)
            self._array_offsets = _cumulative([n for _, n in results])
            if self._label_mask_paths is not None:
                item = self.dtype(0).itemsize
                masks = self.map(lambda p, i: get_file_size(p), _paths=self._label_mask_paths)
                for i, mask_size in enumerate(masks):
                    if self._array_file_sizes[i] // item != mask_size:
                        raise RuntimeError(
                            f"mismatch between size of source file ('{self._array_paths[i]}', "
                            f"{self._array_file_sizes[i] // item:,d}) and size of corresponding label mask file "
                            f"('{self._label_mask_paths[i]}', {mask_size:,d})"
                        )
        return self._array_file_sizes, self._array_offsets

    def _read_chunk_from_array(self, path: PathOrStr, index: int, dtype=None) -> torch.Tensor:
        start = index * self.sequence_length
        return load_array_slice_into_tensor(path, start, start + self.sequence_length, dtype or self.dtype)

    def _usable_instances(self, n_bytes: int, item_size: int) -> int:
        target = self.max_target_sequence_length
        if target is None or target == self.sequence_length:
            return n_bytes // (item_size * self.sequence_length)
        return (n_bytes // (item_size * target)) * (target // self.sequence_length)

    def _get_file_size_and_length(self, path: PathOrStr, idx: int, dtype=None) -> Tuple[int, int]:
        del idx
        size = get_file_size(path)
        return size, self._usable_instances(size, (dtype or self.dtype)(0).itemsize)


class NumpyFSLDatasetMixture(NumpyFSLDataset):
    """Uses ``path_offset_index[(str(path), i)]`` tokens from the ``i``-th path (a sampled source mixture)."""

    def __init__(self, *paths: PathOrStr, path_offset_index: Dict[Tuple[str, int], int], seed: int, **kwargs):
        super().__init__(*paths, **kwargs)
        self._path_offset_index = path_offset_index
        self._seed = seed

    def _get_file_size_and_length(self, path: PathOrStr, idx: int, dtype=None) -> Tuple[int, int]:
        item = (dtype or self.dtype)(0).itemsize
        try:
            size = self._path_offset_index[(str(path), idx)] * self.dtype(0).itemsize
        except KeyError:
            raise OLMoEnvironmentError(f"Item not found in path index @ {(path, idx)}")
        return size, self._usable_instances(size, item)


class NumpyPaddedFSLDataset(NumpyFSLDataset):
    """
    Instances never span documents: each is one document, truncated to ``sequence_length`` and right-padded.
    ``label_mask`` is False on padding. Used for evaluation sets and fine-tuning data.
    """

    indices_dtype: NumpyUIntTypes = np.uint32

    def __init__(self, *paths: PathOrStr, **kwargs):
        kwargs.pop("max_target_sequence_length", None)
        super().__init__(*paths, **kwargs)
        self._array_instance_offsets: Optional[Tuple[Tuple[int, int], ...]] = None
        self._tables: Dict[int, np.ndarray] = {}

    @property
    def offsets(self) -> Tuple[Tuple[int, int], ...]:
        if self._array_instance_offsets is None:
            item = np.dtype(self.indices_dtype).itemsize
            counts = [self._get_instance_indices_path(p).stat().st_size // (2 * item) for p in self.paths]
            self._array_instance_offsets = _cumulative(counts)
        return self._array_instance_offsets

    @property
    def file_sizes(self) -> Tuple[int, ...]:
        if self._array_file_sizes is None:
            self._array_file_sizes = tuple(self.map(lambda p, _: get_file_size(p)))
        return self._array_file_sizes

    def prepare(self) -> None:
        if self.fs_local_rank == 0:
            self._write_instance_indices()
        barrier()
        len(self)

    def _get_instance_indices_path(self, source_path: PathOrStr) -> Path:
        return self._cache_path("instance-indices", source_path, seq=self.sequence_length,
                                dt=np.dtype(self.indices_dtype).name)

    def _write_instance_indices(self) -> None:
        for path in dict.fromkeys(self.paths):
            target = self._get_instance_indices_path(path)
            if target.is_file():
                continue
            log.info(f"Gathering instance indices for '{path}'...")
            _, n = segment_documents_into_instances(path, target, max_sequence_length=self.sequence_length,
                                                    eos_token_id=self.eos_token_id, dtype=self.dtype,
                                                    indices_dtype=self.indices_dtype)
            log.info(f"Created {n:,d} instances of sequence length up to {self.sequence_length} from '{path}'")

    def _bounds(self, src: int, local: int) -> Tuple[int, int]:
        table = self._tables.get(src)
        if table is None:
            table = self._tables[src] = _mmap(self._get_instance_indices_path(self.paths[src]), self.indices_dtype)
        return int(table[2 * local]), int(table[2 * local + 1])

    def _pad(self, item: Dict[str, Any]) -> Dict[str, Any]:
        ids = item["input_ids"]
        n, L = len(ids), self.sequence_length
        mask = torch.zeros(L, dtype=torch.bool)
        mask[:n] = item["label_mask"] if "label_mask" in item else True
        padded = torch.full((L,), self.pad_token_id, dtype=ids.dtype)
        padded[:n] = ids
        item["input_ids"], item["label_mask"] = padded, mask
        return item

    def __getitem__(self, index: int) -> Dict[str, Any]:
        src, local = self._source_of(index)
        start, end = self._bounds(src, local)
        ids = load_array_slice_into_tensor(self.paths[src], start, end, self.dtype)
        item: Dict[str, Any] = {"input_ids": ids}
        if self._label_mask_paths is not None:
            item["label_mask"] = load_array_slice_into_tensor(self._label_mask_paths[src], start, end, np.bool_)
        item = self._pad(item)
        if self.instance_filter_config is not None:
            item["instance_mask"] = self._validate_instance(item["input_ids"], self.instance_filter_config)
        if self._include_instance_metadata:
            item["metadata"] = self._instance_metadata(src)
        if self._generate_doc_lengths:
            item["doc_lens"] = get_document_lengths(item["input_ids"], self.eos_token_id, bos_token_id=self.bos_token_id)
        return item


class NumpyPackedFSLDataset(NumpyFSLDatasetBase):
    """
    Documents are packed whole into instances with the best-fit-decreasing heuristic, so no document is split
    (documents longer than an instance are truncated or fragmented per ``long_doc_strategy``). Packing runs per group
    of ``source_group_size`` consecutive files, treated as one concatenated token stream.
    """

    indices_dtype: NumpyUIntTypes = np.uint64

    def __init__(self, *paths: PathOrStr, long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate,
                 source_group_size: int = 1, **kwargs):
        super().__init__(*paths, **kwargs)
        assert source_group_size >= 1
        self._long_doc_strategy = LongDocStrategy(long_doc_strategy)
        self._source_group_size = source_group_size
        self._groups: List[List[PathOrStr]] = list(chunked(self.paths, source_group_size))
        self._mask_groups = None if self._label_mask_paths is None else list(chunked(self._label_mask_paths, source_group_size))
        self._metadata_groups = list(chunked(self._metadata, source_group_size))
        self._source_sizes: Optional[List[int]] = None
        self._offsets: Optional[Tuple[Tuple[int, int], ...]] = None
        self._starts: Optional[List[int]] = None
        self._tables: Dict[int, Tuple[np.ndarray, np.ndarray, np.ndarray]] = {}

    @property
    def fingerprint_fields(self) -> Tuple[str, ...]:
        return ("vocab_size", "pad_token_id", "eos_token_id", "dtype", "long_doc_strategy", "bos_token_id",
                "sequence_length", "source_group_size")

    @property
    def long_doc_strategy(self) -> LongDocStrategy:
        return self._long_doc_strategy

    @property
    def source_group_size(self) -> int:
        return self._source_group_size

    @property
    def source_sizes(self) -> List[int]:
        """Number of tokens in every source file."""
        if self._source_sizes is None:
            item = self.dtype(0).itemsize
            self._source_sizes = [s // item for s in self.file_sizes]
        return self._source_sizes

    @property
    def source_size_groups(self) -> List[List[int]]:
        """:data:`source_sizes` cut into the groups that are packed together."""
        return list(chunked(self.source_sizes, self._source_group_size))

    def _table_paths(self, group: Sequence[PathOrStr]) -> Tuple[Path, Path, Path]:
        params = dict(seq=self.sequence_length, long=str(self._long_doc_strategy), dt=np.dtype(self.indices_dtype).name)
        return (self._cache_path("document-indices", *group, **params),
                self._cache_path("instance-offsets", *group, **params),
                self._cache_path("documents-by-instance", *group, **params))

    @property
    def source_instance_offsets(self) -> Tuple[Tuple[int, int], ...]:
        if self._offsets is None:
            item = np.dtype(self.indices_dtype).itemsize
            self._offsets = _cumulative([self._table_paths(g)[1].stat().st_size // (2 * item) for g in self._groups])
        return self._offsets

    def prepare(self) -> None:
        if self.fs_local_rank == 0:
            for group in self._groups:
                if not all(p.is_file() for p in self._table_paths(group)):
                    self._pack_group(group)
        barrier()
        len(self)

    def __len__(self) -> int:
        return self.source_instance_offsets[-1][1]

    def _pack_group(self, group: Sequence[PathOrStr]) -> None:
        log.info(f"Packing documents from {list(group)} into instances...")
        L = self.sequence_length
        docs: List[Tuple[int, int]] = []
        base = 0
        item = self.dtype(0).itemsize
        for path in group:
            for start, end in iter_document_indices(path, eos_token_id=self.eos_token_id, dtype=self.dtype,
                                                    bos_token_id=self.bos_token_id):
                if end - start <= L:
                    docs.append((base + start, base + end))
                elif self._long_doc_strategy == LongDocStrategy.truncate:
                    docs.append((base + start, base + start + L))
                else:
                    docs.extend((base + s, base + min(end, s + L)) for s in range(start, end, L))
            base += get_file_size(path) // item
        doc_arr = np.asarray(docs, dtype=self.indices_dtype).reshape(-1, 2)
        instances, doc_arr, total_tokens = InstancePacker(L).pack_documents(doc_arr)
        counts = np.fromiter((len(x) for x in instances), dtype=np.int64, count=len(instances))
        ends = np.cumsum(counts)
        inst_offsets = np.stack([ends - counts, ends], axis=1).astype(self.indices_dtype).reshape(-1)
        docs_by_instance = np.fromiter((d for inst in instances for d in inst), dtype=self.indices_dtype,
                                       count=int(counts.sum()))
        doc_path, off_path, by_path = self._table_paths(group)
        write_array_to_disk(doc_arr.reshape(-1).astype(self.indices_dtype), doc_path)
        write_array_to_disk(docs_by_instance, by_path)
        write_array_to_disk(inst_offsets, off_path)  # last: its presence marks the group as complete
        pad = L * len(instances) - total_tokens
        log.info(f"Packed {total_tokens:,} tokens into {len(instances):,d} instances of length {L:,d} "
                 f"({pad / max(len(instances), 1):.1f} padding tokens per instance on average)")

    def __getitem__(self, index: int) -> Dict[str, Any]:
        offsets = self.source_instance_offsets
        if self._starts is None:
            self._starts = [o[0] for o in offsets]
        g, local = locate(offsets, self._starts, int(index), len(self))
        tables = self._tables.get(g)
        if tables is None:
            tables = self._tables[g] = tuple(_mmap(p, self.indices_dtype) for p in self._table_paths(self._groups[g]))  # type: ignore
        doc_table, inst_offsets, docs_by_instance = tables
        group = self._groups[g]
        first_source = g * self._source_group_size
        sizes = self.source_sizes[first_source: first_source + len(group)]
        masks = None if self._mask_groups is None else self._mask_groups[g]
        L = self.sequence_length
        input_ids = torch.full((L,), self.pad_token_id, dtype=torch.long)
        label_mask = torch.zeros(L, dtype=torch.bool)
        pos = 0
        for doc_id in docs_by_instance[int(inst_offsets[2 * local]): int(inst_offsets[2 * local + 1])]:
            start, end = int(doc_table[2 * int(doc_id)]), int(doc_table[2 * int(doc_id) + 1])
            file_base = 0
            for k, n_tokens in enumerate(sizes):  # which file of the group holds this document
                if start < file_base + n_tokens:
                    break
                file_base += n_tokens
            else:
                raise RuntimeError(f"document {doc_id} lies outside its source group")
            n = end - start
            tokens = load_array_slice_into_tensor(group[k], start - file_base, end - file_base, self.dtype)
            input_ids[pos: pos + n] = tokens
            label_mask[pos: pos + n] = True if masks is None else load_array_slice_into_tensor(
                masks[k], start - file_base, end - file_base, np.bool_)
            pos += n
        out: Dict[str, Any] = {"input_ids": input_ids, "label_mask": label_mask}
        if self.instance_filter_config is not None:
            out["instance_mask"] = self._validate_instance(input_ids, self.instance_filter_config)
        if self._include_instance_metadata:
            out["metadata"] = [dict(m) for m in self._metadata_groups[g]]
        if self._generate_doc_lengths:
            out["doc_lens"] = get_document_lengths(input_ids, self.eos_token_id, bos_token_id=self.bos_token_id)
        return out
