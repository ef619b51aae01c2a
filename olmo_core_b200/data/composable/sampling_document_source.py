"""Module path of src/olmo_core/data/composable/sampling_document_source.py; the classes live in :mod:`.token_source`."""

from .configs import *  # noqa: F401,F403  (attaches the ``Config`` attributes)
from .token_source import SamplingDocumentSource  # noqa: F401
