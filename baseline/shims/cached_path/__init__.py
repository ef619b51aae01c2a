"""Local-files-only stand-in for the `cached_path` package (used by the reference arm of the benchmark)."""

from pathlib import Path

from . import schemes  # noqa: F401


def cached_path(url_or_filename, **kwargs) -> Path:
    p = Path(str(url_or_filename))
    if "://" in str(url_or_filename) and not str(url_or_filename).startswith("file://"):
        raise FileNotFoundError(f"remote paths are not available offline: {url_or_filename}")
    if not p.exists():
        raise FileNotFoundError(str(p))
    return p
