"""Launcher for multi-process tests (module path of src/olmo_core/testing/distributed.py:111-147)."""

from . import run_distributed_test

__all__ = ["run_distributed_test"]
