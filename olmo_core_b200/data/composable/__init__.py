"""
Composable data loading for fixed-sequence-length text (package of src/olmo_core/data/composable/__init__.py)::

    TokenSource  ->  ...  ->  InstanceSource  ->  ...  ->  ComposableDataLoader

* token / document sources give random access to token ids (documents also to their boundaries): in memory, numpy
  files, concatenations, slices, samples and ratio-based mixes;
* instance sources turn them into instances of ``sequence_length`` tokens: concat-and-chunk, document packing, random
  data, and concatenations / slices / samples / mixes of other instance sources;
* the loader shuffles instances globally (or per source, or interleaved), shards batches over data-parallel ranks and
  resumes exactly from its ``state_dict``.

Every source class has its serializable config at ``<Source>.Config``; ``source.visualize()`` prints the tree.
"""

from ..types import LongDocStrategy
from . import (
    concat_and_chunk_instance_source,
    instance_source,
    mixing_document_source,
    mixing_instance_source,
    mixing_token_source,
    packing_instance_source,
    random_instance_source,
    sampling_document_source,
    sampling_instance_source,
    sampling_token_source,
    sliced_instance_source,
    sliced_token_source,
    token_source,
)
from .concat_and_chunk_instance_source import *  # noqa: F401,F403
from .data_loader import ComposableDataLoader, ComposableDataLoaderConfig, InstanceFilterConfig, ShuffleStrategy
from .instance_source import *  # noqa: F401,F403
from .mixing_document_source import *  # noqa: F401,F403
from .mixing_instance_source import *  # noqa: F401,F403
from .mixing_token_source import *  # noqa: F401,F403
from .numpy_document_source import (
    NumpyDocumentSource,
    NumpyDocumentSourceConfig,
    NumpyDocumentSourceConfigBase,
    NumpyDocumentSourceMixConfig,
)
from .packing_instance_source import *  # noqa: F401,F403
from .random_instance_source import *  # noqa: F401,F403
from .sampling_document_source import *  # noqa: F401,F403
from .sampling_instance_source import *  # noqa: F401,F403
from .sampling_token_source import *  # noqa: F401,F403
from .sliced_instance_source import *  # noqa: F401,F403
from .sliced_token_source import *  # noqa: F401,F403
from .source_abc import SourceABC
from .token_source import *  # noqa: F401,F403
from .utils import SEED_NOT_SET, calculate_sample_sizes, reset_composable_seed, resolve_seed, set_composable_seed
from .visualize import render_source, visualize_source

_source_modules = (
    token_source, sliced_token_source, sampling_token_source, sampling_document_source, mixing_token_source,
    mixing_document_source, instance_source, concat_and_chunk_instance_source, packing_instance_source,
    random_instance_source, sliced_instance_source, sampling_instance_source, mixing_instance_source,
)

__all__ = [
    "SourceABC", "NumpyDocumentSource", "NumpyDocumentSourceConfig", "NumpyDocumentSourceMixConfig",
    "NumpyDocumentSourceConfigBase", "LongDocStrategy",
    "ComposableDataLoader", "ComposableDataLoaderConfig", "InstanceFilterConfig", "ShuffleStrategy", "SEED_NOT_SET",
    "calculate_sample_sizes", "set_composable_seed", "reset_composable_seed", "resolve_seed", "render_source",
    "visualize_source", *[name for module in _source_modules for name in module.__all__],
]
