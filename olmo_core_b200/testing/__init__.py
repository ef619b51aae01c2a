"""
Helpers for the test-suite (package of src/olmo_core/testing/__init__.py): pytest marks and parametrisations for
devices / backends in :mod:`.utils`, the launcher for multi-process tests in :mod:`.distributed`.
"""

from .distributed import run_distributed_test
from .utils import *  # noqa: F401,F403
from .utils import __all__ as _util_names

__all__ = ["run_distributed_test", *_util_names]
