"""
Variable-sequence-length data ("dataset decomposition", arXiv:2405.13226)
(behaviour of src/olmo_core/data/numpy_dataset.py:1620-2300).

Every document is cut into pieces whose lengths are powers of two between ``min_sequence_length`` and
``max_sequence_length`` (largest first); pieces of equal length form a *bucket*. A batch holds pieces of one bucket only
-- always the same number of tokens, no padding, no cross-document attention -- and a *curriculum* decides in which
order batches of the different buckets are visited.
"""

from __future__ import annotations

import hashlib
import logging
import math
from abc import abstractmethod
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ...aliases import PathOrStr
from ...config import Config, StrEnum
from ...distributed.utils import barrier
from ...exceptions import OLMoConfigurationError
from ...io import get_file_size
from ..types import NumpyUIntTypes
from ..utils import (
    bucket_documents,
    chunk_array,
    divide_into_buckets,
    get_doc_lengths_from_indices,
    get_rng,
    load_array_slice_into_tensor,
    write_array_to_disk,
)
from .base import InstanceFilterConfig, NumpyDatasetBase, locate

log = logging.getLogger(__name__)

__all__ = ["VSLCurriculum", "VSLNaturalCurriculum", "VSLGrowthCurriculum", "VSLGrowP2Curriculum",
           "VSLGrowLinearCurriculum", "VSLCurriculumType", "VSLCurriculumConfig", "NumpyVSLDataset"]

Buckets = Sequence[Tuple[int, int]]  # (sequence length, number of batches), shortest first


class VSLCurriculum:
    """Decides how many batches each bucket contributes and the order in which batches are visited."""

    @abstractmethod
    def batches_per_bucket(self, dataset: "NumpyVSLDataset", global_batch_size: int) -> List[Tuple[int, int]]:
        raise NotImplementedError

    @abstractmethod
    def get_batch_indices(self, batches_per_bucket: Buckets, seed: int) -> np.ndarray:
        """A permutation of ``range(total batches)``; batch ids count through the buckets from the shortest up."""
        raise NotImplementedError

    def get_total_batches(self, batches_per_bucket: Buckets) -> int:
        return sum(n for _, n in batches_per_bucket)

    def log_buckets(self, dataset: "NumpyVSLDataset", global_batch_size: int, batches_per_bucket: Buckets) -> None:
        natural = VSLNaturalCurriculum().batches_per_bucket(dataset, global_batch_size)
        for i, (seq_len, n) in enumerate(batches_per_bucket):
            extra = f" used ({natural[i][1]:d} total)" if n != natural[i][1] else ""
            log.info(f"- bucket {i}:   sequence length {seq_len:>6d} => {n:>6d} batches{extra}")

    @property
    @abstractmethod
    def short_str(self) -> str:
        """Identifier used in cache file names."""
        raise NotImplementedError

    @staticmethod
    def _long_batch_first(indices: np.ndarray, pick: int) -> None:
        """Swap batch ``indices[pick]`` to the front: starting with the longest bucket surfaces memory problems at step 1."""
        indices[0], indices[pick] = indices[pick], indices[0]


@dataclass
class VSLNaturalCurriculum(VSLCurriculum):
    """Uniformly shuffled batches: every bucket is visited in proportion to its size throughout training."""

    def batches_per_bucket(self, dataset: "NumpyVSLDataset", global_batch_size: int) -> List[Tuple[int, int]]:
        return [(seq_len, n // (global_batch_size // seq_len)) for seq_len, n in dataset.instances_per_bucket]

    def get_batch_indices(self, batches_per_bucket: Buckets, seed: int) -> np.ndarray:
        total = self.get_total_batches(batches_per_bucket)
        indices = np.arange(total, dtype=np.uint32)
        rng = get_rng(seed)
        self._long_batch_first(indices, int(rng.integers(total - batches_per_bucket[-1][1], total)))
        rng.shuffle(indices[1:])
        return indices

    @property
    def short_str(self) -> str:
        return "vsl-natural"


@dataclass
class VSLGrowthCurriculum(VSLCurriculum):
    """
    ``num_cycles`` cycles; within a cycle there is one sub-cycle per bucket and the share of each bucket shifts from
    sub-cycle to sub-cycle according to the subclass's odds, from mostly short to mostly long sequences.
    """

    num_cycles: int = 8
    balanced: bool = False
    """Use the same number of batches from every bucket (drops data from the larger buckets)."""

    def batches_per_bucket(self, dataset: "NumpyVSLDataset", global_batch_size: int) -> List[Tuple[int, int]]:
        natural = VSLNaturalCurriculum().batches_per_bucket(dataset, global_batch_size)
        if self.balanced:
            smallest = min(n for _, n in natural)
            return [(seq_len, self.num_cycles * (smallest // self.num_cycles)) for seq_len, _ in natural]
        return [(seq_len, self.num_cycles * (n // self.num_cycles)) for seq_len, n in natural]

    def get_cycle_distribution(self, indices: np.ndarray, batches_per_bucket: Buckets, cycle: int = 0) -> List[List[int]]:
        """For each sub-cycle of ``cycle``, how many of its batches come from each bucket."""
        length = indices.shape[0] // self.num_cycles
        edges = np.cumsum([0] + [n for _, n in batches_per_bucket])
        return [
            [int(((sub >= lo) & (sub < hi)).sum()) for lo, hi in zip(edges[:-1], edges[1:])]
            for sub in np.array_split(indices[cycle * length: (cycle + 1) * length], len(batches_per_bucket))
        ]

    def get_batch_indices(self, batches_per_bucket: Buckets, seed: int) -> np.ndarray:
        assert batches_per_bucket[0][0] < batches_per_bucket[-1][0]
        rng = get_rng(seed)
        n_buckets = len(batches_per_bucket)
        starts = np.cumsum([0] + [n for _, n in batches_per_bucket])
        cycles: List[np.ndarray] = []
        for cycle in range(self.num_cycles):
            # batches of every bucket that belong to this cycle, split over the sub-cycles by the bucket's odds
            per_bucket: List[List[np.ndarray]] = []
            for b, (_, n) in enumerate(batches_per_bucket):
                per_cycle = divide_into_buckets(n, self.num_cycles)
                mine = chunk_array(np.arange(n, dtype=np.uint32), per_cycle)[cycle] + np.uint32(starts[b])
                per_bucket.append(chunk_array(mine, self._get_num_bucket_batches_for_cycle(b, n_buckets, per_cycle[cycle])))
            for sub in range(n_buckets):
                mixed = np.concatenate([per_bucket[b][sub] for b in range(n_buckets)])
                rng.shuffle(mixed)
                cycles.append(mixed)
        indices = np.concatenate(cycles)
        self._long_batch_first(indices, int(np.argmax(indices >= starts[-2])))
        assert indices.shape[0] == self.get_total_batches(batches_per_bucket)
        return indices

    @classmethod
    @abstractmethod
    def _get_bucket_odds_for_cycle(cls, bucket_idx: int, num_buckets: int) -> List[int]:
        raise NotImplementedError

    @classmethod
    def _ramp(cls, bucket_idx: int, num_buckets: int) -> List[int]:
        """Weight exponent of a bucket per sub-cycle: rises to ``num_buckets`` and then falls back."""
        start = num_buckets - bucket_idx
        return [start + c if start + c <= num_buckets else start - ((start + c) % num_buckets) for c in range(num_buckets)]

    @classmethod
    def _get_num_bucket_batches_for_cycle(cls, bucket_idx: int, num_buckets: int, num_batches: int) -> List[int]:
        odds = cls._get_bucket_odds_for_cycle(bucket_idx, num_buckets)
        total_odds = sum(odds)
        counts = [round(o / total_odds * num_batches) for o in odds]
        if sum(counts) < num_batches:
            counts[-1] += num_batches - sum(counts)
        return counts

    def _suffix(self) -> str:
        return f"{self.num_cycles}-cycle{'-balanced' if self.balanced else ''}"


@dataclass
class VSLGrowP2Curriculum(VSLGrowthCurriculum):
    """"Grow-P2": bucket weights are powers of two of the ramp."""

    @classmethod
    def _get_bucket_odds_for_cycle(cls, bucket_idx: int, num_buckets: int) -> List[int]:
        return [2 ** (e - 1) for e in cls._ramp(bucket_idx, num_buckets)]

    @property
    def short_str(self) -> str:
        return f"vsl-grow-p2-{self._suffix()}"


@dataclass
class VSLGrowLinearCurriculum(VSLGrowthCurriculum):
    """"Grow-Linear": bucket weights are the ramp itself."""

    @classmethod
    def _get_bucket_odds_for_cycle(cls, bucket_idx: int, num_buckets: int) -> List[int]:
        return cls._ramp(bucket_idx, num_buckets)

    @property
    def short_str(self) -> str:
        return f"vsl-grow-linear-{self._suffix()}"


class VSLCurriculumType(StrEnum):
    natural = "natural"
    grow_p2 = "grow_p2"
    grow_linear = "grow_linear"


@dataclass
class VSLCurriculumConfig(Config):
    name: VSLCurriculumType = VSLCurriculumType.natural
    num_cycles: Optional[int] = None
    balanced: Optional[bool] = None

    def validate(self) -> None:
        if self.name == VSLCurriculumType.natural:
            self.num_cycles = None
            self.balanced = None

    def build(self) -> VSLCurriculum:
        if self.name == VSLCurriculumType.natural:
            if self.num_cycles is not None or self.balanced is not None:
                raise OLMoConfigurationError(f"'num_cycles' and 'balanced' are not valid for the {self.name} curriculum")
            return VSLNaturalCurriculum()
        if self.num_cycles is None or self.balanced is None:
            raise OLMoConfigurationError(f"'num_cycles' and 'balanced' are required for the {self.name} curriculum")
        cls = VSLGrowP2Curriculum if self.name == VSLCurriculumType.grow_p2 else VSLGrowLinearCurriculum
        return cls(num_cycles=self.num_cycles, balanced=self.balanced)


def _is_pow2(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


class NumpyVSLDataset(NumpyDatasetBase, torch.utils.data.Dataset):
    indices_dtype: NumpyUIntTypes = np.uint32

    def __init__(self, *paths: PathOrStr, pad_token_id: int, eos_token_id: int, vocab_size: int, max_sequence_length: int,
                 min_sequence_length: int = 256, curriculum: Optional[VSLCurriculum] = None,
                 dtype: NumpyUIntTypes = np.uint16, metadata: Optional[Union[List[Dict[str, Any]], Dict[str, Any]]] = None,
                 include_instance_metadata: Optional[bool] = None,
                 instance_filter_config: Optional[InstanceFilterConfig] = None):
        if not _is_pow2(max_sequence_length):
            raise OLMoConfigurationError("'max_sequence_length' must be a power of 2")
        if not _is_pow2(min_sequence_length):
            raise OLMoConfigurationError("'min_sequence_length' must be a power of 2")
        if max_sequence_length <= min_sequence_length:
            raise OLMoConfigurationError("'max_sequence_length' should be bigger than 'min_sequence_length'")
        if include_instance_metadata is None and metadata:
            include_instance_metadata = True
        if isinstance(metadata, list):
            if len(metadata) != len(paths):
                raise OLMoConfigurationError("'metadata' should have the same length as the number of file paths")
        else:
            metadata = [metadata or {}] * len(paths)
        super().__init__(*paths, pad_token_id=pad_token_id, eos_token_id=eos_token_id, vocab_size=vocab_size, dtype=dtype)
        self._metadata = metadata
        self._include_instance_metadata = bool(include_instance_metadata)
        self._max_sequence_length = max_sequence_length
        self._min_sequence_length = min_sequence_length
        self._curriculum = curriculum or VSLNaturalCurriculum()
        self.instance_filter_config = instance_filter_config
        self._array_offsets: Optional[Tuple[Tuple[int, int], ...]] = None
        self._starts: Optional[List[int]] = None
        self._instances_per_bucket: Optional[Tuple[Tuple[int, int], ...]] = None
        self._tables: Dict[int, np.ndarray] = {}

    @property
    def fingerprint_fields(self) -> Tuple[str, ...]:
        return ("vocab_size", "pad_token_id", "eos_token_id", "dtype", "min_sequence_length", "max_sequence_length",
                "curriculum")

    @property
    def max_sequence_length(self) -> int:
        return self._max_sequence_length

    @property
    def min_sequence_length(self) -> int:
        return self._min_sequence_length

    @property
    def curriculum(self) -> VSLCurriculum:
        return self._curriculum

    @property
    def all_sequence_lengths(self) -> List[int]:
        lo, hi = int(math.log2(self.min_sequence_length)), int(math.log2(self.max_sequence_length))
        return [2**e for e in range(lo, hi + 1)]

    @property
    def lengths_dtype(self) -> NumpyUIntTypes:
        for dt in (np.uint8, np.uint16, np.uint32, np.uint64):
            if self.max_sequence_length - 1 <= np.iinfo(dt).max:
                return dt
        raise RuntimeError("unreachable")

    # -- cached tables -----------------------------------------------------------------------------------------
    def _get_document_indices_path(self, path: PathOrStr) -> Path:
        h = hashlib.sha256()
        h.update(str(path).encode())
        h.update(str(get_file_size(path)).encode())
        for seq_len in self.all_sequence_lengths:
            h.update(str(seq_len).encode())
        return self.work_dir / "dataset-common" / f"bucketed-doc-indices-{h.hexdigest()}.npy"

    def _get_instance_lengths_path(self) -> Path:
        return self.work_dir / f"dataset-{self.fingerprint}" / "instance-lengths.npy"

    def _get_instance_bucket_path(self, seq_len: int) -> Path:
        return self.work_dir / f"dataset-{self.fingerprint}" / f"bucket{seq_len}-indices.npy"

    @property
    def offsets(self) -> Tuple[Tuple[int, int], ...]:
        if self._array_offsets is None:
            item = np.dtype(self.indices_dtype).itemsize
            out, start = [], 0
            for path in self.paths:
                n = self._get_document_indices_path(path).stat().st_size // (2 * item)
                out.append((start, start + n))
                start += n
            self._array_offsets = tuple(out)
        return self._array_offsets

    def prepare(self) -> None:
        if self.fs_local_rank == 0:
            for path in dict.fromkeys(self.paths):
                target = self._get_document_indices_path(path)
                if not target.is_file():
                    n_docs, n_pieces = bucket_documents(path, target, buckets=self.all_sequence_lengths,
                                                        eos_token_id=self.eos_token_id, dtype=self.dtype,
                                                        indices_dtype=self.indices_dtype)
                    log.info(f"Created {n_pieces:,d} bucketed documents from {n_docs:,d} original documents in '{path}'")
            lengths_path = self._get_instance_lengths_path()
            if not lengths_path.is_file():
                lengths = np.zeros(len(self), dtype=self.lengths_dtype)
                for path, (lo, hi) in zip(self.paths, self.offsets):
                    table = np.memmap(self._get_document_indices_path(path), dtype=self.indices_dtype, mode="r")
                    lengths[lo:hi] = get_doc_lengths_from_indices(table)
                write_array_to_disk(lengths, lengths_path)
            lengths = self.get_instance_lengths()
            for seq_len in self.all_sequence_lengths:
                bucket_path = self._get_instance_bucket_path(seq_len)
                if not bucket_path.is_file():
                    write_array_to_disk(np.nonzero(lengths == seq_len)[0].astype(self.indices_dtype), bucket_path)
        barrier()
        len(self)

    def __len__(self) -> int:
        return self.offsets[-1][1]

    def __getitem__(self, index: int) -> Dict[str, Any]:
        offsets = self.offsets
        if self._starts is None:
            self._starts = [o[0] for o in offsets]
        src, local = locate(offsets, self._starts, int(index), len(self))
        table = self._tables.get(src)
        if table is None:
            table = self._tables[src] = np.memmap(self._get_document_indices_path(self.paths[src]),
                                                  dtype=self.indices_dtype, mode="r")
        input_ids = load_array_slice_into_tensor(self.paths[src], int(table[2 * local]), int(table[2 * local + 1]), self.dtype)
        out: Dict[str, Any] = {"input_ids": input_ids}
        if self.instance_filter_config is not None:
            out["instance_mask"] = self._validate_instance(input_ids, self.instance_filter_config)
        if self._include_instance_metadata:
            out["metadata"] = dict(self._metadata[src])
        return out

    def get_instance_lengths(self) -> np.ndarray:
        """Memory-mapped length of every instance."""
        return np.memmap(self._get_instance_lengths_path(), dtype=self.lengths_dtype, mode="r")

    def get_instance_bucket(self, seq_len: int) -> np.ndarray:
        """Memory-mapped indices of the instances of length ``seq_len``."""
        path = self._get_instance_bucket_path(seq_len)
        if path.stat().st_size == 0:
            return np.zeros(0, dtype=self.indices_dtype)
        return np.memmap(path, dtype=self.indices_dtype, mode="r")

    def get_instance_buckets(self) -> List[Tuple[int, np.ndarray]]:
        return [(s, self.get_instance_bucket(s)) for s in self.all_sequence_lengths]

    @property
    def instances_per_bucket(self) -> Tuple[Tuple[int, int], ...]:
        if self._instances_per_bucket is None:
            item = np.dtype(self.indices_dtype).itemsize
            self._instances_per_bucket = tuple(
                (s, self._get_instance_bucket_path(s).stat().st_size // item) for s in self.all_sequence_lengths)
        return self._instances_per_bucket
