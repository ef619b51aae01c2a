"""
Document source over flat token files, the format written by the dolma toolkit
(API of src/olmo_core/data/composable/numpy_document_source.py:1-593): each ``.npy`` path is a headerless array of
token ids; an optional ``.csv.gz`` beside it lists document boundaries, otherwise boundaries are found by scanning for
the EOS (or BOS) token once and cached under the work dir.
"""

from __future__ import annotations

import hashlib
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np

from ...aliases import PathOrStr
from ...config import Config
from ...exceptions import OLMoConfigurationError
from ...io import get_file_size, glob_directory, is_url, join_path, normalize_path
from ..mixes import DataMix, DataMixBase
from ..tokenizer import TokenizerConfig
from ..types import NumpyDatasetDType
from ..utils import iter_document_indices, load_array_slice
from .token_source import DocumentSource, TokenRange

__all__ = ["NumpyDocumentSource", "NumpyDocumentSourceConfig", "NumpyDocumentSourceMixConfig"]


def _dtype_for(tokenizer: TokenizerConfig, dtype: Optional[NumpyDatasetDType]):
    if dtype is not None:
        return NumpyDatasetDType(dtype).as_np_dtype()
    for candidate in (np.uint8, np.uint16, np.uint32, np.uint64):
        if tokenizer.vocab_size - 1 <= np.iinfo(candidate).max:
            return candidate
    raise ValueError("vocab size too large")


def _expand(patterns: Sequence[PathOrStr]) -> List[str]:
    out: List[str] = []
    for p in patterns:
        p = str(p)
        if "*" in p:
            matches = sorted(glob_directory(p))
            if not matches:
                raise FileNotFoundError(f"pattern '{p}' did not match any files")
            out.extend(matches)
        else:
            out.append(normalize_path(p))
    return out


class NumpyDocumentSource(DocumentSource):
    DISPLAY_ICON = ""

    def __init__(self, *, source_paths: Sequence[PathOrStr], dtype, work_dir: PathOrStr, tokenizer: TokenizerConfig,
                 label_mask_paths: Optional[Sequence[PathOrStr]] = None, label: Optional[str] = None):
        super().__init__(work_dir=work_dir, label=label)
        if not source_paths:
            raise OLMoConfigurationError("At least one source path is required.")
        if label_mask_paths is not None and len(label_mask_paths) != len(source_paths):
            raise OLMoConfigurationError("'label_mask_paths' must match 'source_paths' one to one")
        self._paths = tuple(normalize_path(p) for p in source_paths)
        self._mask_paths = None if label_mask_paths is None else tuple(normalize_path(p) for p in label_mask_paths)
        self._dtype = dtype
        self._tokenizer = tokenizer
        item = np.dtype(dtype).itemsize
        with ThreadPoolExecutor(max_workers=min(16, len(self._paths))) as pool:
            sizes = list(pool.map(get_file_size, self._paths))
        self._sizes = np.array([s // item for s in sizes], dtype=np.int64)
        self._ends = np.cumsum(self._sizes)

    Config: type

    def __repr__(self) -> str:
        return f"NumpyDocumentSource{self._paths!r}"

    @property
    def source_paths(self) -> Tuple[str, ...]:
        return self._paths

    @property
    def eos_token_id(self) -> int:
        return self._tokenizer.eos_token_id

    @property
    def bos_token_id(self) -> Optional[int]:
        return self._tokenizer.bos_token_id

    @property
    def fingerprint(self) -> str:
        h = hashlib.sha256(f"class=NumpyDocumentSource,dtype={np.dtype(self._dtype).name},".encode())
        for p, n in zip(self._paths, self._sizes.tolist()):
            h.update(f"{p}:{n},".encode())
        for p in self._mask_paths or ():
            h.update(f"mask={p},".encode())
        return h.hexdigest()

    @property
    def num_tokens(self) -> int:
        return int(self._ends[-1])

    def children(self):
        return []

    def get_token_range(self, start_idx: int, end_idx: int) -> TokenRange:
        start_idx, end_idx = self.validate_indices(start_idx, end_idx)
        ids, masks = [], []
        pos = start_idx
        i = int(np.searchsorted(self._ends, start_idx, side="right"))
        while pos < end_idx:
            base = int(self._ends[i]) - int(self._sizes[i])
            lo, hi = pos - base, min(int(self._sizes[i]), end_idx - base)
            ids.append(load_array_slice(self._paths[i], lo, hi, self._dtype))
            if self._mask_paths is not None:
                masks.append(load_array_slice(self._mask_paths[i], lo, hi, np.bool_))
            pos += hi - lo
            i += 1
        out: TokenRange = {"input_ids": np.concatenate(ids) if len(ids) != 1 else ids[0]}
        if masks:
            out["label_mask"] = np.concatenate(masks) if len(masks) != 1 else masks[0]
        return out

    def _offsets_cache(self, path: str) -> Path:
        name = hashlib.sha256(f"{path},{self.eos_token_id},{self.bos_token_id}".encode()).hexdigest()[:24]
        return self.work_dir / f"doc-offsets-{name}.npy"

    def _file_offsets(self, path: str) -> np.ndarray:
        cache = self._offsets_cache(path)
        if cache.is_file():
            return np.load(cache)
        offsets = np.array(list(iter_document_indices(path, eos_token_id=self.eos_token_id, dtype=self._dtype)),
                           dtype=np.int64).reshape(-1, 2)
        if self.fs_local_rank == 0:
            cache.parent.mkdir(parents=True, exist_ok=True)
            tmp = cache.with_suffix(".tmp.npy")
            np.save(tmp, offsets)
            tmp.replace(cache)
        return offsets

    def get_document_offsets(self) -> Iterable[Tuple[int, int]]:
        base = 0
        for path, n in zip(self._paths, self._sizes.tolist()):
            for s, e in self._file_offsets(path).tolist():
                yield base + s, base + e
            base += n


@dataclass
class NumpyDocumentSourceConfig(Config):
    """``source_paths`` may hold glob patterns; files are grouped ``source_group_size`` at a time into sources."""

    source_paths: List[str]
    tokenizer: TokenizerConfig
    dtype: Optional[NumpyDatasetDType] = None
    label_mask_paths: Optional[List[str]] = None
    source_group_size: int = 1
    label: Optional[str] = None

    @classmethod
    def from_source_groups(cls, source_groups: Dict[str, List[str]], *, tokenizer: TokenizerConfig,
                           **kwargs) -> Dict[str, "NumpyDocumentSourceConfig"]:
        """One config per labelled group of paths."""
        return {label: cls(source_paths=list(paths), tokenizer=tokenizer, label=label, **kwargs)
                for label, paths in source_groups.items()}

    def build(self, work_dir: PathOrStr) -> List[NumpyDocumentSource]:
        paths = _expand(self.source_paths)
        masks = None if self.label_mask_paths is None else _expand(self.label_mask_paths)
        if masks is not None and len(masks) != len(paths):
            raise OLMoConfigurationError("'label_mask_paths' must match 'source_paths' one to one after globbing")
        dtype = _dtype_for(self.tokenizer, self.dtype)
        g = max(1, self.source_group_size)
        return [NumpyDocumentSource(source_paths=paths[i:i + g], dtype=dtype, work_dir=work_dir, tokenizer=self.tokenizer,
                                    label_mask_paths=None if masks is None else masks[i:i + g], label=self.label)
                for i in range(0, len(paths), g)]


@dataclass
class NumpyDocumentSourceMixConfig(Config):
    """Sources for a named data mix (a manifest of ``label,relative/path`` lines resolved under ``mix_base_dir``)."""

    tokenizer: TokenizerConfig
    mix: Union[str, DataMixBase]
    mix_base_dir: str
    dtype: Optional[NumpyDatasetDType] = None
    source_group_size: int = 1

    def build(self, work_dir: PathOrStr) -> List[NumpyDocumentSource]:
        if self.tokenizer.identifier is None:
            raise OLMoConfigurationError("Missing tokenizer identifier required to construct data mix")
        mix = self.mix if isinstance(self.mix, DataMixBase) else DataMix(self.mix)
        paths, labels = mix.build(self.mix_base_dir, self.tokenizer.identifier)
        dtype = _dtype_for(self.tokenizer, self.dtype)
        by_label: Dict[str, List[str]] = {}
        for p, l in zip(paths, labels):
            by_label.setdefault(l, []).append(p)
        g = max(1, self.source_group_size)
        out: List[NumpyDocumentSource] = []
        for label, group in by_label.items():
            group = _expand(group)
            out += [NumpyDocumentSource(source_paths=group[i:i + g], dtype=dtype, work_dir=work_dir,
                                        tokenizer=self.tokenizer, label=label) for i in range(0, len(group), g)]
        return out


NumpyDocumentSource.Config = NumpyDocumentSourceConfig
