"""
Opt-in persistent memoisation on the filesystem (role of src/olmo_core/fs_cache.py:23-96).

``@maybe_cache()`` behaves like ``functools.cache`` when the environment variable ``OLMO_CORE_FS_CACHE_DIR`` names a
directory, and is a no-op otherwise. Results are pickled to ``<dir>/<qualname>-<sha256 of arguments>.pkl``; a file lock
per key makes concurrent ranks compute a value once, and the file appears atomically (write to a temp name, fsync,
rename), so a reader never sees a half-written pickle.
"""

from __future__ import annotations

import dataclasses
import functools
import hashlib
import json
import logging
import os
import pickle
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Optional, TypeVar

from filelock import FileLock

log = logging.getLogger(__name__)

__all__ = ["CACHE_DIR_ENV_VAR", "maybe_cache"]

CACHE_DIR_ENV_VAR = "OLMO_CORE_FS_CACHE_DIR"

F = TypeVar("F", bound=Callable[..., Any])


def _canonical(obj: Any) -> Any:
    """Reduce arguments to JSON types so that equal arguments always hash equally."""
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {"__dc__": type(obj).__qualname__, **{f.name: _canonical(getattr(obj, f.name)) for f in dataclasses.fields(obj)}}
    if isinstance(obj, Enum):
        return _canonical(obj.value)
    if isinstance(obj, dict):
        return {str(k): _canonical(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_canonical(v) for v in obj]
    if isinstance(obj, (set, frozenset)):
        return sorted(_canonical(v) for v in obj)
    if isinstance(obj, Path):
        return str(obj)
    if obj is None or isinstance(obj, (bool, int, float, str)):
        return obj
    raise TypeError(f"argument of type {type(obj).__name__} cannot be used as a cache key")


def _deterministic_hash(obj: Any) -> str:
    return hashlib.sha256(json.dumps(_canonical(obj), sort_keys=True).encode("utf-8")).hexdigest()


def _store(path: Path, value: Any) -> None:
    tmp = path.with_name(f"{path.name}.{os.getpid()}.tmp")
    try:
        with tmp.open("wb") as f:
            pickle.dump(value, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    finally:
        tmp.unlink(missing_ok=True)


def maybe_cache(*, condition: Optional[Callable[..., bool]] = None) -> Callable[[F], F]:
    """
    Cache a function's result on disk when ``OLMO_CORE_FS_CACHE_DIR`` is set (and ``condition(*args, **kwargs)`` holds,
    if given). Arguments must reduce to JSON; results must pickle.
    """

    def decorator(fn: F) -> F:
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            root = os.environ.get(CACHE_DIR_ENV_VAR)
            if root is None or (condition is not None and not condition(*args, **kwargs)):
                return fn(*args, **kwargs)
            cache_dir = Path(root)
            cache_dir.mkdir(parents=True, exist_ok=True)
            key = f"{fn.__qualname__}-{_deterministic_hash((args, kwargs))}"
            target = cache_dir / f"{key}.pkl"
            with FileLock(str(cache_dir / f"{key}.lock")):
                if target.exists():
                    log.debug("filesystem cache hit for %s()", fn.__qualname__)
                    with target.open("rb") as f:
                        return pickle.load(f)
                log.debug("filesystem cache miss for %s()", fn.__qualname__)
                value = fn(*args, **kwargs)
                _store(target, value)
                return value

        return wrapper  # type: ignore[return-value]

    return decorator
