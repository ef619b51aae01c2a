"""
Base classes of datasets backed by token-id ``.npy`` files (flat arrays of unsigned ints, local or remote)
(interface of src/olmo_core/data/numpy_dataset.py:100-450).

A dataset is a read-only view: ``dataset[i]`` reads one instance with a ranged read of exactly its bytes, so
petabyte-scale collections are never loaded or even fully downloaded. Everything derived from the data (document
boundaries, packing tables, length buckets) is computed once in :meth:`prepare` by the first rank of each
file-system and cached under ``work_dir``, keyed by a hash of the source path and the parameters.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
from abc import ABC, abstractmethod
from bisect import bisect_right
from copy import deepcopy
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, TypeVar, Union

import numpy as np
import torch

from ...aliases import PathOrStr
from ...config import Config
from ...distributed.utils import get_fs_local_rank
from ...exceptions import OLMoConfigurationError
from ...io import _client, get_file_size, is_url, normalize_path
from ..types import NumpyUIntTypes
from ..utils import find_periodic_sequences

T = TypeVar("T")

__all__ = ["InstanceFilterConfig", "NumpyDatasetBase", "NumpyFSLDatasetBase", "locate"]


@dataclass
class InstanceFilterConfig(Config):
    """Marks instances that contain a token pattern of period in ``[min, max]`` repeated ``max_count`` times or more."""

    repetition_max_period: int = 13
    repetition_min_period: int = 1
    repetition_max_count: int = 32


def locate(offsets: Sequence[Tuple[int, int]], starts: Sequence[int], index: int, size: int) -> Tuple[int, int]:
    """``(source number, index within source)`` of global instance ``index`` given cumulative ``(start, end)`` offsets."""
    pos = index if index >= 0 else size + index
    if not 0 <= pos < size:
        raise IndexError(f"{index} is out of bounds for dataset of size {size}")
    i = bisect_right(starts, pos) - 1
    while offsets[i][1] <= pos:  # skip empty sources
        i += 1
    return i, pos - offsets[i][0]


class NumpyDatasetBase(ABC):
    def __init__(self, *paths: PathOrStr, pad_token_id: int, eos_token_id: int, vocab_size: int,
                 dtype: NumpyUIntTypes = np.uint16, bos_token_id: Optional[int] = None):
        if not paths:
            raise OLMoConfigurationError("At least one path is required")
        self._array_paths = tuple(paths)
        self._pad_token_id = pad_token_id
        self._eos_token_id = eos_token_id
        self._bos_token_id = bos_token_id
        self._vocab_size = vocab_size
        self._dtype = dtype
        self._fs_local_rank = get_fs_local_rank()
        self._work_dir: Optional[Path] = None
        self._work_dir_set = False
        self._array_file_sizes: Optional[Tuple[int, ...]] = None

    # -- description ------------------------------------------------------------------------------------
    @property
    @abstractmethod
    def max_sequence_length(self) -> int:
        raise NotImplementedError

    @property
    def paths(self) -> Tuple[PathOrStr, ...]:
        return self._array_paths

    @property
    def file_sizes(self) -> Tuple[int, ...]:
        """Size in bytes of every source file."""
        if self._array_file_sizes is None:
            self._array_file_sizes = tuple(self.map(lambda path, _: get_file_size(path)))
        return self._array_file_sizes

    @property
    def pad_token_id(self) -> int:
        return self._pad_token_id

    @property
    def eos_token_id(self) -> int:
        return self._eos_token_id

    @property
    def bos_token_id(self) -> Optional[int]:
        return self._bos_token_id

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    @property
    def dtype(self) -> NumpyUIntTypes:
        return self._dtype

    @property
    def num_tokens(self) -> int:
        raise NotImplementedError

    # -- fingerprint: detects that a restored run reads different data -------------------------------------
    @property
    def fingerprint_version(self) -> str:
        return "v2.0"

    @property
    def fingerprint_fields(self) -> Tuple[str, ...]:
        return ("vocab_size", "pad_token_id", "eos_token_id", "dtype", "bos_token_id")

    @property
    def fingerprint(self) -> str:
        h = hashlib.sha256()
        h.update(f"class={self.__class__.__name__}".encode())
        for name in self.fingerprint_fields:
            h.update(f"{name}={getattr(self, name)},".encode())
        for path, size in zip(self.paths, self.file_sizes):
            h.update(f"path={os.path.basename(str(path))},size={size},".encode())
        return h.hexdigest()

    # -- environment --------------------------------------------------------------------------------------
    @property
    def fs_local_rank(self) -> int:
        return self._fs_local_rank

    @fs_local_rank.setter
    def fs_local_rank(self, fs_local_rank: int) -> None:
        self._fs_local_rank = fs_local_rank

    @property
    def work_dir(self) -> Path:
        if self._work_dir is not None:
            return self._work_dir
        import tempfile

        return Path(tempfile.gettempdir())

    @work_dir.setter
    def work_dir(self, work_dir: PathOrStr) -> None:
        if is_url(work_dir):
            raise OLMoConfigurationError("'work_dir' must be a local directory")
        self._work_dir = Path(normalize_path(work_dir))
        self._work_dir_set = True

    @property
    def work_dir_set(self) -> bool:
        return self._work_dir_set

    def map(self, func: Callable[[PathOrStr, int], T], *, max_workers: Optional[int] = None, method: str = "threads",
            _paths: Optional[Sequence[PathOrStr]] = None) -> List[T]:
        """``[func(path, i) for i, path in enumerate(paths)]`` evaluated concurrently; results in path order."""
        paths = _paths or self.paths
        if max_workers == 0 or len(paths) == 1:
            return [func(p, i) for i, p in enumerate(paths)]
        if method == "threads":
            for p in {str(p).split("://")[0] for p in paths if is_url(p)}:
                _client(f"{p}://")  # create each remote client once, before the threads race for it
            pool_cls: Any = concurrent.futures.ThreadPoolExecutor
        elif method == "processes":
            pool_cls = concurrent.futures.ProcessPoolExecutor
        else:
            raise ValueError(method)
        with pool_cls(max_workers=max_workers) as pool:
            futures = [pool.submit(func, p, i) for i, p in enumerate(paths)]
        return [f.result() for f in futures]

    def prepare(self) -> None:
        """Build cached index files. Set :data:`work_dir` first; call from the main process, on every rank."""

    @abstractmethod
    def __len__(self) -> int:
        raise NotImplementedError

    @abstractmethod
    def __getitem__(self, index: int) -> Dict[str, Any]:
        """An instance: at least ``input_ids`` (integer tensor)."""
        raise NotImplementedError

    def _validate_instance(self, input_ids: torch.Tensor, cfg: InstanceFilterConfig) -> bool:
        for m in find_periodic_sequences(input_ids.numpy(), max_period=cfg.repetition_max_period,
                                         min_period=cfg.repetition_min_period):
            if m.times >= cfg.repetition_max_count:
                return False
        return True

    def _cache_path(self, kind: str, *sources: PathOrStr, **params) -> Path:
        """Where a derived index for ``sources`` with ``params`` is cached under the work directory."""
        h = hashlib.sha256()
        for s in sources:
            h.update(str(s).encode())
        tag = "-".join(f"{k}{v}" for k, v in sorted(params.items()))
        return self.work_dir / "dataset-common" / f"{kind}-{tag}-{h.hexdigest()}.npy"


class NumpyFSLDatasetBase(NumpyDatasetBase, torch.utils.data.Dataset):
    """Common state of the fixed-sequence-length datasets."""

    def __init__(self, *paths: PathOrStr, sequence_length: int, pad_token_id: int, eos_token_id: int, vocab_size: int,
                 dtype: NumpyUIntTypes = np.uint16, metadata: Optional[Union[List[Dict[str, Any]], Dict[str, Any]]] = None,
                 include_instance_metadata: Optional[bool] = None, generate_doc_lengths: bool = False,
                 bos_token_id: Optional[int] = None, instance_filter_config: Optional[InstanceFilterConfig] = None,
                 label_mask_paths: Optional[Sequence[PathOrStr]] = None):
        if include_instance_metadata is None and metadata:
            include_instance_metadata = True
        if isinstance(metadata, list):
            if len(metadata) != len(paths):
                raise OLMoConfigurationError("'metadata' should have the same length as the number of file paths")
        else:
            metadata = [metadata or {}] * len(paths)
        if label_mask_paths is not None and len(label_mask_paths) != len(paths):
            raise OLMoConfigurationError("There must be the same number of 'label_mask_paths' as there are 'paths'")
        super().__init__(*paths, pad_token_id=pad_token_id, eos_token_id=eos_token_id, vocab_size=vocab_size, dtype=dtype,
                         bos_token_id=bos_token_id)
        self._metadata = tuple(metadata)
        self._sequence_length = sequence_length
        self._include_instance_metadata = bool(include_instance_metadata)
        self._generate_doc_lengths = generate_doc_lengths
        self.instance_filter_config = instance_filter_config
        self._label_mask_paths = tuple(label_mask_paths) if label_mask_paths is not None else None

    @property
    def sequence_length(self) -> int:
        return self._sequence_length

    @property
    def max_sequence_length(self) -> int:
        return self._sequence_length

    @property
    def max_target_sequence_length(self) -> Optional[int]:
        return None

    @property
    def metadata(self) -> Tuple[Dict[str, Any], ...]:
        return self._metadata

    def _instance_metadata(self, source: int) -> Dict[str, Any]:
        return deepcopy(self._metadata[source])
