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

from .configs import *  # noqa: F401,F403
from .configs import __all__ as _config_names
from .data_loader import ComposableDataLoader, ComposableDataLoaderConfig, InstanceFilterConfig, ShuffleStrategy
from .instance_source import *  # noqa: F401,F403
from .instance_source import __all__ as _instance_names
from ..types import LongDocStrategy
from .numpy_document_source import (
    NumpyDocumentSource,
    NumpyDocumentSourceConfig,
    NumpyDocumentSourceConfigBase,
    NumpyDocumentSourceMixConfig,
)
from .source_abc import SourceABC
from .token_source import *  # noqa: F401,F403
from .token_source import __all__ as _token_names
from .utils import SEED_NOT_SET, calculate_sample_sizes, reset_composable_seed, resolve_seed, set_composable_seed
from .visualize import render_source, visualize_source

__all__ = [
    "SourceABC", "NumpyDocumentSource", "NumpyDocumentSourceConfig", "NumpyDocumentSourceMixConfig",
    "NumpyDocumentSourceConfigBase", "LongDocStrategy",
    "ComposableDataLoader", "ComposableDataLoaderConfig", "InstanceFilterConfig", "ShuffleStrategy", "SEED_NOT_SET",
    "calculate_sample_sizes", "set_composable_seed", "reset_composable_seed", "resolve_seed", "render_source",
    "visualize_source", *_token_names, *_instance_names, *_config_names,
]
