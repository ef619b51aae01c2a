"""
Serialisable builders of the numpy datasets (fields of src/olmo_core/data/numpy_dataset.py:2306-2826).

Every config names its token files either explicitly (``paths``, optionally globs) or through a data ``mix`` under
``mix_base_dir``; labels of a mix become per-file ``metadata``.
"""

from __future__ import annotations

import logging
import random
from abc import ABC, abstractmethod
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Type, TypeVar, Union

import numpy as np

from ...aliases import PathOrStr
from ...config import Config
from ...exceptions import OLMoConfigurationError
from ...io import glob_directory
from ..mixes import DataMix, DataMixBase
from ..source_mixture import SourceMixtureDatasetConfig
from ..tokenizer import TokenizerConfig
from ..types import LongDocStrategy, NumpyDatasetDType, NumpyUIntTypes
from .base import InstanceFilterConfig, NumpyDatasetBase
from .fsl import NumpyFSLDataset, NumpyFSLDatasetMixture, NumpyPackedFSLDataset, NumpyPaddedFSLDataset
from .interleaved import NumpyInterleavedFSLDataset
from .vsl import NumpyVSLDataset, VSLCurriculumConfig

log = logging.getLogger(__name__)

__all__ = ["NumpyDatasetConfig", "NumpyFSLDatasetConfig", "NumpyPaddedFSLDatasetConfig", "NumpyPackedFSLDatasetConfig",
           "NumpyInterleavedFSLDatasetConfig", "NumpyVSLDatasetConfig"]

C = TypeVar("C", bound="NumpyDatasetConfig")


@dataclass
class NumpyDatasetConfig(Config, ABC):
    tokenizer: TokenizerConfig
    paths: Optional[List[str]] = None
    mix: Optional[Union[str, DataMixBase]] = None
    mix_base_dir: Optional[str] = None
    expand_glob: bool = False
    dtype: Optional[NumpyDatasetDType] = None
    """Storage type of the token files; by default the smallest unsigned type that holds the vocabulary."""
    metadata: Optional[List[Dict[str, Any]]] = None
    include_instance_metadata: bool = True
    instance_filter_config: Optional[InstanceFilterConfig] = None
    source_permutation_seed: Optional[int] = None
    """Shuffle the order of the source files with this seed before building the dataset."""
    work_dir: Optional[str] = None
    """Where derived index files are cached; share it between runs to avoid recomputing them."""
    ignore_fingerprint_mismatch: bool = False

    @abstractmethod
    def build(self) -> NumpyDatasetBase:
        raise NotImplementedError

    def get_dtype(self) -> NumpyUIntTypes:
        if self.dtype is not None:
            return NumpyDatasetDType(self.dtype).as_np_dtype()
        for dt in NumpyDatasetDType:
            if self.tokenizer.vocab_size - 1 <= np.iinfo(dt.as_np_dtype()).max:
                log.info(f"Assuming dtype '{dt}' based on vocab size")
                return dt.as_np_dtype()
        raise ValueError("vocab size too big!")

    @staticmethod
    def _expand_globs(patterns: Sequence[str]) -> List[str]:
        out: List[str] = []
        for pattern in patterns:
            matches = sorted(glob_directory(pattern))
            if not matches:
                raise FileNotFoundError(f"Pattern '{pattern}' did not match any files")
            out.extend(matches)
        return out

    def _resolve_paths_metadata(self, *, allow_mix: bool, label_mask_paths: Optional[Sequence[PathOrStr]] = None
                                ) -> Tuple[List[str], Optional[List[Dict[str, Any]]], Optional[List[PathOrStr]]]:
        if self.paths is not None and self.mix is not None:
            raise OLMoConfigurationError("Only one of 'paths' or 'mix' can be set")
        metadata = self.metadata
        masks: Optional[List[PathOrStr]] = None if label_mask_paths is None else [str(p) for p in label_mask_paths]
        if self.paths is not None:
            paths = [str(p) for p in self.paths]
            if self.expand_glob:
                paths = self._expand_globs(paths)
                if masks is not None:
                    masks = list(self._expand_globs([str(m) for m in masks]))
        else:
            if self.mix is None:
                raise OLMoConfigurationError("Either 'paths' or 'mix' must be set")
            if not allow_mix:
                raise OLMoConfigurationError("'mix' is not supported for this dataset type")
            if self.mix_base_dir is None:
                raise OLMoConfigurationError("'mix_base_dir' is required to build a dataset from a mix")
            if self.tokenizer.identifier is None:
                raise OLMoConfigurationError("Missing tokenizer identifier required to construct data mix")
            mix = self.mix if isinstance(self.mix, DataMixBase) else DataMix(self.mix)
            paths, labels = mix.build(self.mix_base_dir, self.tokenizer.identifier)
            paths = [str(p) for p in paths]
            if metadata is None:
                metadata = [{"label": label} for label in labels]
        if self.source_permutation_seed is not None:
            order = list(range(len(paths)))
            random.Random(self.source_permutation_seed).shuffle(order)
            paths = [paths[i] for i in order]
            metadata = None if metadata is None else [metadata[i] for i in order]
            masks = None if masks is None else [masks[i] for i in order]
        return paths, metadata, masks

    def _common(self) -> Dict[str, Any]:
        tok = self.tokenizer
        return dict(pad_token_id=tok.pad_token_id, eos_token_id=tok.eos_token_id, vocab_size=tok.vocab_size,
                    dtype=self.get_dtype(), include_instance_metadata=self.include_instance_metadata,
                    instance_filter_config=self.instance_filter_config)

    def _finalize(self, dataset: NumpyDatasetBase) -> NumpyDatasetBase:
        if self.work_dir is not None:
            dataset.work_dir = Path(self.work_dir)
        return dataset

    @classmethod
    def glob(cls: Type[C], *glob_paths: str, **kwargs: Any) -> C:
        """A config whose paths are glob patterns, expanded (and required to match) when the dataset is built."""
        return cls(paths=list(glob_paths), mix=None, mix_base_dir=None, expand_glob=True, **kwargs)

    @classmethod
    def from_data_mix(cls: Type[C], mix: Union[str, DataMixBase], *, tokenizer: TokenizerConfig, **kwargs: Any) -> C:
        if tokenizer.identifier is None:
            raise OLMoConfigurationError("Missing tokenizer identifier required to construct data mix")
        return cls(mix=mix, paths=None, tokenizer=tokenizer, **kwargs)


@dataclass(kw_only=True)
class NumpyFSLDatasetConfig(NumpyDatasetConfig):
    sequence_length: int
    max_target_sequence_length: Optional[int] = None
    """Largest sequence length later stages of the run will use (keeps the token order identical across stages)."""
    generate_doc_lengths: bool = False
    label_mask_paths: Optional[List[str]] = None
    source_mixture_config: Optional[SourceMixtureDatasetConfig] = None

    @classmethod
    def from_src_mix(cls, src_mix: SourceMixtureDatasetConfig, **kwargs: Any) -> "NumpyFSLDatasetConfig":
        return cls(source_mixture_config=src_mix, paths=None, mix=None, mix_base_dir=None, **kwargs)

    def validate(self) -> None:
        if self.sequence_length <= 0:
            raise OLMoConfigurationError("'sequence_length' must be positive")
        if self.source_mixture_config is not None:
            if self.paths is not None or self.mix is not None:
                raise OLMoConfigurationError("Specify only one of 'paths', 'mix', or 'source_mixture_config'")
            if self.label_mask_paths is not None:
                raise OLMoConfigurationError("'label_mask_paths' is not supported alongside 'source_mixture_config'")

    def build(self) -> NumpyDatasetBase:
        self.validate()
        shared = dict(self._common(), sequence_length=self.sequence_length,
                      max_target_sequence_length=self.max_target_sequence_length,
                      generate_doc_lengths=self.generate_doc_lengths, bos_token_id=self.tokenizer.bos_token_id)
        if self.source_mixture_config is not None:
            mixture = self.source_mixture_config.build(npdtype=self.get_dtype(), sequence_length=self.sequence_length)
            return self._finalize(NumpyFSLDatasetMixture(
                *mixture.to_paths(), seed=self.source_mixture_config.seed, path_offset_index=mixture.to_index(),
                metadata=self.metadata, **shared))
        paths, metadata, masks = self._resolve_paths_metadata(allow_mix=True, label_mask_paths=self.label_mask_paths)
        return self._finalize(NumpyFSLDataset(*paths, metadata=metadata, label_mask_paths=masks, **shared))


@dataclass(kw_only=True)
class NumpyPaddedFSLDatasetConfig(NumpyDatasetConfig):
    sequence_length: int
    label_mask_paths: Optional[List[str]] = None

    def validate(self) -> None:
        if self.sequence_length <= 0:
            raise OLMoConfigurationError("'sequence_length' must be positive")

    def build(self) -> NumpyDatasetBase:
        self.validate()
        paths, metadata, masks = self._resolve_paths_metadata(allow_mix=True, label_mask_paths=self.label_mask_paths)
        return self._finalize(NumpyPaddedFSLDataset(
            *paths, sequence_length=self.sequence_length, metadata=metadata, label_mask_paths=masks,
            bos_token_id=self.tokenizer.bos_token_id, **self._common()))


@dataclass(kw_only=True)
class NumpyPackedFSLDatasetConfig(NumpyDatasetConfig):
    sequence_length: int
    generate_doc_lengths: bool = False
    label_mask_paths: Optional[List[str]] = None
    long_doc_strategy: LongDocStrategy = LongDocStrategy.truncate
    source_group_size: int = 1
    """Number of consecutive source files packed together (more files per group: tighter packing, more memory)."""

    def validate(self) -> None:
        if self.sequence_length <= 0:
            raise OLMoConfigurationError("'sequence_length' must be positive")
        if self.source_group_size < 1:
            raise OLMoConfigurationError("'source_group_size' must be at least 1")

    def build(self) -> NumpyDatasetBase:
        self.validate()
        paths, metadata, masks = self._resolve_paths_metadata(allow_mix=True, label_mask_paths=self.label_mask_paths)
        return self._finalize(NumpyPackedFSLDataset(
            *paths, sequence_length=self.sequence_length, metadata=metadata, label_mask_paths=masks,
            generate_doc_lengths=self.generate_doc_lengths, bos_token_id=self.tokenizer.bos_token_id,
            long_doc_strategy=self.long_doc_strategy, source_group_size=self.source_group_size, **self._common()))


@dataclass(kw_only=True)
class NumpyInterleavedFSLDatasetConfig(NumpyDatasetConfig):
    sequence_length: int
    docs_per_instance: int
    chunks_per_doc: int
    seed: int
    label_mask_paths: Optional[List[str]] = None
    interleaving_exempt_paths: Optional[List[str]] = None

    def validate(self) -> None:
        for name in ("sequence_length", "docs_per_instance", "chunks_per_doc"):
            if getattr(self, name) <= 0:
                raise OLMoConfigurationError(f"'{name}' must be positive")

    def build(self) -> NumpyDatasetBase:
        self.validate()
        paths, metadata, masks = self._resolve_paths_metadata(allow_mix=True, label_mask_paths=self.label_mask_paths)
        exempt = self.interleaving_exempt_paths
        if exempt is not None and self.expand_glob:
            exempt = self._expand_globs(exempt)
        return self._finalize(NumpyInterleavedFSLDataset(
            *paths, sequence_length=self.sequence_length, seed=self.seed, docs_per_instance=self.docs_per_instance,
            chunks_per_doc=self.chunks_per_doc, metadata=metadata, label_mask_paths=masks,
            bos_token_id=self.tokenizer.bos_token_id, interleaving_exempt_paths=exempt, **self._common()))


@dataclass(kw_only=True)
class NumpyVSLDatasetConfig(NumpyDatasetConfig):
    max_sequence_length: int
    min_sequence_length: int
    vsl_curriculum: Optional[VSLCurriculumConfig] = None

    def validate(self) -> None:
        if self.max_sequence_length <= 0:
            raise OLMoConfigurationError("'max_sequence_length' must be positive")
        if self.min_sequence_length <= 0:
            raise OLMoConfigurationError("'min_sequence_length' must be positive")
        if self.min_sequence_length > self.max_sequence_length:
            raise OLMoConfigurationError("'min_sequence_length' cannot be larger than 'max_sequence_length'")
        if self.tokenizer.bos_token_id is not None:
            raise OLMoConfigurationError("'bos_token_id' is not supported for the VSL dataset")
        if self.vsl_curriculum is not None:
            self.vsl_curriculum.validate()

    def build(self) -> NumpyDatasetBase:
        self.validate()
        paths, metadata, _ = self._resolve_paths_metadata(allow_mix=True)
        return self._finalize(NumpyVSLDataset(
            *paths, max_sequence_length=self.max_sequence_length, min_sequence_length=self.min_sequence_length,
            curriculum=None if self.vsl_curriculum is None else self.vsl_curriculum.build(), metadata=metadata,
            **self._common()))
