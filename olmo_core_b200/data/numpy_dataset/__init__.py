"""
Datasets over token-id ``.npy`` files and their config builders (public names of src/olmo_core/data/numpy_dataset.py).
"""

from .base import InstanceFilterConfig, NumpyDatasetBase, NumpyFSLDatasetBase
from .config import (
    NumpyDatasetConfig,
    NumpyFSLDatasetConfig,
    NumpyInterleavedFSLDatasetConfig,
    NumpyPackedFSLDatasetConfig,
    NumpyPaddedFSLDatasetConfig,
    NumpyVSLDatasetConfig,
)
from .fsl import NumpyFSLDataset, NumpyFSLDatasetMixture, NumpyPackedFSLDataset, NumpyPaddedFSLDataset
from .interleaved import NumpyInterleavedFSLDataset
from .vsl import (
    NumpyVSLDataset,
    VSLCurriculum,
    VSLCurriculumConfig,
    VSLCurriculumType,
    VSLGrowLinearCurriculum,
    VSLGrowP2Curriculum,
    VSLGrowthCurriculum,
    VSLNaturalCurriculum,
)

__all__ = [
    "NumpyDatasetBase",
    "NumpyFSLDatasetBase",
    "NumpyFSLDataset",
    "NumpyFSLDatasetMixture",
    "NumpyPaddedFSLDataset",
    "NumpyPackedFSLDataset",
    "NumpyInterleavedFSLDataset",
    "NumpyVSLDataset",
    "VSLCurriculum",
    "VSLNaturalCurriculum",
    "VSLGrowthCurriculum",
    "VSLGrowP2Curriculum",
    "VSLGrowLinearCurriculum",
    "VSLCurriculumType",
    "VSLCurriculumConfig",
    "NumpyDatasetConfig",
    "NumpyFSLDatasetConfig",
    "NumpyPaddedFSLDatasetConfig",
    "NumpyPackedFSLDatasetConfig",
    "NumpyInterleavedFSLDatasetConfig",
    "NumpyVSLDatasetConfig",
    "InstanceFilterConfig",
]
