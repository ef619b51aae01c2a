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
from ..types import LongDocStrategy, NumpyDatasetDType
from ..utils import iter_document_indices, load_array_slice
from .token_source import DocumentSource, DocumentSourceConfig, TokenRange

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
                 label_mask_paths: Optional[Sequence[PathOrStr]] = None, label: Optional[str] = None,
                 max_document_length: Optional[int] = None,
                 long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate,
                 _source_sizes: Optional[Sequence[int]] = None, _label_mask_sizes: Optional[Sequence[int]] = None):
        super().__init__(work_dir=work_dir, label=label)
        self._max_document_length = max_document_length
        self._long_doc_strategy = LongDocStrategy(long_doc_strategy)
        if not source_paths:
            raise OLMoConfigurationError("At least one source path is required.")
        if label_mask_paths is not None and len(label_mask_paths) != len(source_paths):
            raise OLMoConfigurationError("'label_mask_paths' must match 'source_paths' one to one")
        self._paths = tuple(normalize_path(p) for p in source_paths)
        self._mask_paths = None if label_mask_paths is None else tuple(normalize_path(p) for p in label_mask_paths)
        self._dtype = dtype
        self._tokenizer = tokenizer
        # File sizes are given by a parent that was split (no second look at the files) or read here, in parallel.
        def items(paths: Tuple[str, ...], item: int) -> List[int]:
            with ThreadPoolExecutor(max_workers=min(16, len(paths))) as pool:
                return [n // item for n in pool.map(get_file_size, paths)]

        sizes = list(_source_sizes) if _source_sizes is not None else items(self._paths, np.dtype(dtype).itemsize)
        if len(sizes) != len(self._paths):
            raise OLMoConfigurationError("'_source_sizes' must match 'source_paths' one to one")
        self._sizes = np.array(sizes, dtype=np.int64)
        self._ends = np.cumsum(self._sizes)
        self._mask_sizes: Optional[Tuple[int, ...]] = None
        if self._mask_paths is not None:
            mask_sizes = list(_label_mask_sizes) if _label_mask_sizes is not None else items(self._mask_paths, 1)
            self._mask_sizes = tuple(int(n) for n in mask_sizes)
            for mp, mn, sp, sn in zip(self._mask_paths, self._mask_sizes, self._paths, sizes):
                if mn != sn:
                    raise OLMoConfigurationError(
                        "Each file in 'label_mask_paths' should have the same number of items as the corresponding "
                        f"file in 'source_paths', but found {mn:,d} in '{mp}' vs {sn:,d} in '{sp}'.")

    Config: type

    def __repr__(self) -> str:
        return f"NumpyDocumentSource{self._paths!r}"

    @property
    def source_paths(self) -> Tuple[str, ...]:
        return self._paths

    @property
    def source_sizes(self) -> Tuple[int, ...]:
        """Tokens in each source file."""
        return tuple(int(n) for n in self._sizes)

    @property
    def label_mask_paths(self) -> Optional[Tuple[str, ...]]:
        return self._mask_paths

    @property
    def label_mask_sizes(self) -> Optional[Tuple[int, ...]]:
        return self._mask_sizes

    @property
    def dtype(self):
        return self._dtype

    @property
    def tokenizer(self) -> TokenizerConfig:
        return self._tokenizer

    def split_by_source(self, group_size: int = 1) -> List["NumpyDocumentSource"]:
        """One source per ``group_size`` consecutive files
        (src/olmo_core/data/composable/numpy_document_source.py:478-512)."""
        assert group_size >= 1
        out: List[NumpyDocumentSource] = []
        for i in range(0, len(self._paths), group_size):
            sel = slice(i, i + group_size)
            out.append(self.__class__(
                source_paths=self._paths[sel], dtype=self._dtype, work_dir=self.work_dir, tokenizer=self._tokenizer,
                label_mask_paths=None if self._mask_paths is None else self._mask_paths[sel], label=self.label,
                max_document_length=self._max_document_length, long_doc_strategy=self._long_doc_strategy,
                _source_sizes=self.source_sizes[sel],
                _label_mask_sizes=None if self._mask_sizes is None else self._mask_sizes[sel]))
        return out

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
        if self._max_document_length is not None:
            h.update(f"max_document_length={self._max_document_length},{self._long_doc_strategy},".encode())
        return h.hexdigest()

    @property
    def max_document_length(self) -> Optional[int]:
        return self._max_document_length

    @property
    def long_doc_strategy(self) -> LongDocStrategy:
        return self._long_doc_strategy

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
        # Documents longer than ``max_document_length`` are cut to their first part (truncate) or into consecutive
        # parts (fragment), as in src/olmo_core/data/utils.py:253-285. The end of a file always ends a document.
        base, limit = 0, self._max_document_length
        for path, n in zip(self._paths, self._sizes.tolist()):
            last = 0
            for s, e in self._file_offsets(path).tolist():
                if limit is None or e - s <= limit:
                    yield base + s, base + e
                elif self._long_doc_strategy == LongDocStrategy.truncate:
                    yield base + s, base + s + limit
                else:
                    for start in range(s, e, limit):
                        yield base + start, base + min(e, start + limit)
                last = e
            if last != n:
                yield base + last, base + n
            base += n


@dataclass(kw_only=True)
class NumpyDocumentSourceConfigBase(DocumentSourceConfig):
    """What :class:`NumpyDocumentSourceConfig` and :class:`NumpyDocumentSourceMixConfig` share
    (src/olmo_core/data/composable/numpy_document_source.py:33-77)."""

    tokenizer: TokenizerConfig
    dtype: Optional[NumpyDatasetDType] = None
    source_permutation_seed: Optional[int] = None
    """Shuffles the source files before they are grouped into sources."""
    source_group_size: int = 1
    """Number of files per source; ``-1`` puts all files into one source."""
    label: Optional[str] = None
    max_document_length: Optional[int] = None
    """Longer documents are truncated or fragmented (``long_doc_strategy``) when documents are iterated."""
    long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate

    def __post_init__(self):
        if self.source_group_size < -1 or self.source_group_size == 0:
            raise OLMoConfigurationError("'source_group_size' must be -1 or a positive integer.")

    def get_dtype(self):
        return _dtype_for(self.tokenizer, self.dtype)

    def _grouped(self, paths: List[str], masks: Optional[List[str]]):
        """Files (and their masks) in source order, cut into groups."""
        order = list(range(len(paths)))
        if self.source_permutation_seed is not None:
            order = np.random.default_rng(self.source_permutation_seed).permutation(len(paths)).tolist()
        paths = [paths[i] for i in order]
        masks = None if masks is None else [masks[i] for i in order]
        g = len(paths) if self.source_group_size == -1 else self.source_group_size
        for i in range(0, len(paths), max(1, g)):
            yield paths[i:i + g], None if masks is None else masks[i:i + g]

    def _source(self, paths, masks, work_dir, label) -> "NumpyDocumentSource":
        return NumpyDocumentSource(source_paths=paths, dtype=self.get_dtype(), work_dir=work_dir, tokenizer=self.tokenizer,
                                   label_mask_paths=masks, label=label, max_document_length=self.max_document_length,
                                   long_doc_strategy=self.long_doc_strategy)


@dataclass(kw_only=True)
class NumpyDocumentSourceConfig(NumpyDocumentSourceConfigBase):
    """``source_paths`` may hold glob patterns; files are grouped ``source_group_size`` at a time into sources."""

    source_paths: List[str]
    label_mask_paths: Optional[List[str]] = None
    expand_glob: Optional[bool] = None

    @classmethod
    def from_source_groups(cls, source_groups: Dict[str, List[str]], *, tokenizer: TokenizerConfig,
                           **kwargs) -> Dict[str, "NumpyDocumentSourceConfig"]:
        """One config per labelled group of paths."""
        return {label: cls(source_paths=list(paths), tokenizer=tokenizer, label=label, **kwargs)
                for label, paths in source_groups.items()}

    def get_num_tokens(self) -> int:
        """Tokens over all source files, from their sizes alone."""
        item = np.dtype(self.get_dtype()).itemsize
        paths = _expand(self.source_paths)
        with ThreadPoolExecutor(max_workers=min(16, max(1, len(paths)))) as pool:
            return sum(n // item for n in pool.map(get_file_size, paths))

    def build(self, work_dir: PathOrStr) -> List[NumpyDocumentSource]:
        paths = _expand(self.source_paths)
        masks = None if self.label_mask_paths is None else _expand(self.label_mask_paths)
        if masks is not None and len(masks) != len(paths):
            raise OLMoConfigurationError("'label_mask_paths' must match 'source_paths' one to one after globbing")
        return [self._source(ps, ms, work_dir, self.label) for ps, ms in self._grouped(paths, masks)]


@dataclass(kw_only=True)
class NumpyDocumentSourceMixConfig(NumpyDocumentSourceConfigBase):
    """Sources for a named data mix (a manifest of ``label,relative/path`` lines resolved under ``mix_base_dir``)."""

    mix: Union[str, DataMixBase]
    mix_base_dir: str

    def build(self, work_dir: PathOrStr) -> List[NumpyDocumentSource]:
        if self.tokenizer.identifier is None:
            raise OLMoConfigurationError("Missing tokenizer identifier required to construct data mix")
        mix = self.mix if isinstance(self.mix, DataMixBase) else DataMix(self.mix)
        paths, labels = mix.build(self.mix_base_dir, self.tokenizer.identifier)
        by_label: Dict[str, List[str]] = {}
        for p, l in zip(paths, labels):
            by_label.setdefault(l, []).append(p)
        out: List[NumpyDocumentSource] = []
        for label, group in by_label.items():
            out += [self._source(ps, None, work_dir, label) for ps, _ in self._grouped(_expand(group), None)]
        return out


NumpyDocumentSource.Config = NumpyDocumentSourceConfig
