"""
Datasets, data loaders and their config builders for the trainer (public names of src/olmo_core/data/__init__.py).

Text data is prepared as token ids in flat ``.npy`` files. Build a dataset with one of the
:class:`~olmo_core_b200.data.numpy_dataset.NumpyDatasetConfig` builders, or compose one with
:mod:`olmo_core_b200.data.composable`, wrap it with :class:`~olmo_core_b200.data.data_loader.NumpyDataLoaderConfig` and
pass the loader to ``TrainerConfig.build``.
"""

from .collator import DataCollator, PaddingDirection
from .data_loader import (
    DataLoaderBase,
    DataLoaderConfig,
    NumpyDataLoaderBase,
    NumpyDataLoaderConfig,
    NumpyFSLDataLoader,
    NumpyVSLDataLoader,
    TextDataLoaderBase,
)
from .mixes import DataMix, DataMixBase
from .numpy_dataset import (
    InstanceFilterConfig,
    NumpyDatasetBase,
    NumpyDatasetConfig,
    NumpyFSLDataset,
    NumpyFSLDatasetBase,
    NumpyFSLDatasetConfig,
    NumpyFSLDatasetMixture,
    NumpyInterleavedFSLDataset,
    NumpyInterleavedFSLDatasetConfig,
    NumpyPackedFSLDataset,
    NumpyPackedFSLDatasetConfig,
    NumpyPaddedFSLDataset,
    NumpyPaddedFSLDatasetConfig,
    NumpyVSLDataset,
    NumpyVSLDatasetConfig,
    VSLCurriculum,
    VSLCurriculumConfig,
    VSLCurriculumType,
    VSLGrowLinearCurriculum,
    VSLGrowP2Curriculum,
    VSLGrowthCurriculum,
    VSLNaturalCurriculum,
)
from .source_mixture import SourceMixtureConfig, SourceMixtureDatasetConfig, SourceMixtureList
from .tokenizer import TokenizerConfig, TokenizerName
from .types import LongDocStrategy, NumpyDatasetDType

from . import composable  # noqa: E402,F401

__all__ = [
    "composable",
    "NumpyDatasetBase", "NumpyFSLDatasetBase", "NumpyFSLDataset", "NumpyFSLDatasetMixture", "NumpyPaddedFSLDataset",
    "NumpyPackedFSLDataset", "NumpyInterleavedFSLDataset", "NumpyVSLDataset", "VSLCurriculum", "VSLNaturalCurriculum",
    "VSLGrowthCurriculum", "VSLGrowP2Curriculum", "VSLGrowLinearCurriculum", "NumpyDatasetConfig", "NumpyFSLDatasetConfig",
    "NumpyPaddedFSLDatasetConfig", "NumpyPackedFSLDatasetConfig", "NumpyInterleavedFSLDatasetConfig",
    "NumpyVSLDatasetConfig", "InstanceFilterConfig", "VSLCurriculumType", "VSLCurriculumConfig", "NumpyDatasetDType",
    "TokenizerConfig", "TokenizerName", "DataMixBase", "DataMix", "DataCollator", "PaddingDirection", "DataLoaderBase",
    "DataLoaderConfig", "TextDataLoaderBase", "NumpyDataLoaderBase", "NumpyFSLDataLoader", "NumpyVSLDataLoader",
    "NumpyDataLoaderConfig", "LongDocStrategy", "SourceMixtureConfig", "SourceMixtureList", "SourceMixtureDatasetConfig",
]
