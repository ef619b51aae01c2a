"""Module path of src/olmo_core/data/composable/sliced_instance_source.py; the classes live in :mod:`.instance_source`."""

from .configs import *  # noqa: F401,F403  (attaches the ``Config`` attributes)
from .instance_source import SlicedInstanceSource  # noqa: F401
