"""
Uniform file API over local paths and URLs.

Local paths and ``file://`` URLs are handled natively; ``http(s)://`` is read-only through
``requests``; object stores (``s3://``, ``r2://``, ``weka://``, ``gs://``) go through a small
``SchemeClient`` plug-in registry whose default clients import ``boto3`` / ``google.cloud.storage``
lazily and raise :class:`OLMoEnvironmentError` when those are not installed. The function names match
the reference's src/olmo_core/io.py:43-508 so calling code ports unchanged.
"""

from __future__ import annotations

import functools
import io
import logging
import os
import pickle
import random
import re
import shutil
import time
from pathlib import Path
from typing import Any, Callable, Dict, Generator, List, Optional, Tuple, Type, Union
from urllib.parse import urlparse

import torch

from .aliases import PathOrStr
from .exceptions import OLMoEnvironmentError, OLMoInvalidRangeRequestError, OLMoNetworkError

log = logging.getLogger(__name__)

__all__ = [
    "normalize_path",
    "resource_path",
    "join_path",
    "is_url",
    "file_exists",
    "dir_is_empty",
    "get_file_size",
    "get_bytes_range",
    "read_bytes",
    "read_text",
    "upload",
    "copy_file",
    "copy_dir",
    "remove_file",
    "clear_directory",
    "list_directory",
    "glob_directory",
    "deterministic_glob_directory",
    "init_client",
    "deserialize_from_tensor",
    "serialize_to_tensor",
    "retriable",
    "add_cached_path_clients",
    "SchemeClient",
    "register_scheme_client",
    "get_parent",
    "write_bytes",
    "write_text",
]

_URL_RE = re.compile(r"^[a-z0-9]+://.+")


def is_url(path: PathOrStr) -> bool:
    return bool(_URL_RE.match(str(path)))


def normalize_path(path: PathOrStr) -> str:
    """String form of ``path`` without trailing slashes or a ``file://`` prefix."""
    p = str(path).rstrip("/")
    if p.startswith("file://"):
        p = p[len("file://"):]
    return p


def join_path(path: PathOrStr, *paths: PathOrStr) -> PathOrStr:
    """Join two or more paths / URL parts; a single argument is returned as is."""
    for p in paths:
        if is_url(path):
            path = f"{str(path).rstrip('/')}/{str(p).lstrip('/')}"
        else:
            path = Path(path) / p
    return path


def get_parent(path: PathOrStr) -> PathOrStr:
    if is_url(path):
        return str(path).rstrip("/").rsplit("/", 1)[0]
    return Path(path).parent


def retriable(
    max_attempts: int = 3,
    retriable_errors: Tuple[Type[Exception], ...] = (OLMoNetworkError, ConnectionError, TimeoutError),
    backoff: float = 0.5,
    retry_condition: Optional[Callable[[Exception], bool]] = None,
) -> Callable:
    """Retry a function with exponential back-off and jitter on the given error types, or on any error for which
    ``retry_condition`` holds. The last failure is raised as :class:`OLMoNetworkError` (a type that a data-loader
    worker can re-raise from its message alone)."""

    def deco(fn: Callable) -> Callable:
        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            attempt = 0
            while True:
                attempt += 1
                try:
                    return fn(*args, **kwargs)
                except Exception as e:
                    if not (isinstance(e, retriable_errors) or (retry_condition is not None and retry_condition(e))):
                        raise
                    if attempt >= max_attempts:
                        if isinstance(e, OLMoNetworkError):
                            raise
                        raise OLMoNetworkError(f"'{fn.__name__}' failed {max_attempts} attempts with: {e}") from e
                    delay = backoff * (2 ** (attempt - 1)) * (1 + random.random())
                    log.warning("%s failed (%s); retry %d/%d in %.1fs", fn.__name__, e, attempt, max_attempts, delay)
                    time.sleep(delay)

        return wrapped

    return deco


# ----------------------------------------------------------------------------------------------
# scheme clients
# ----------------------------------------------------------------------------------------------


class SchemeClient:
    """Interface an object-store back end implements to be usable through this module."""

    scheme: str = ""

    def exists(self, url: str) -> bool:
        raise NotImplementedError

    def size(self, url: str) -> int:
        raise NotImplementedError

    def read_range(self, url: str, start: int, length: int) -> bytes:
        raise NotImplementedError

    def upload(self, source: Path, url: str, overwrite: bool) -> None:
        raise NotImplementedError

    def delete(self, url: str) -> None:
        raise NotImplementedError

    def list(self, url: str, recurse: bool) -> List[str]:
        raise NotImplementedError


_CLIENTS: Dict[str, SchemeClient] = {}
_CLIENT_FACTORIES: Dict[str, Callable[[], SchemeClient]] = {}


def register_scheme_client(scheme: str, factory: Callable[[], SchemeClient]) -> None:
    _CLIENT_FACTORIES[scheme] = factory
    _CLIENTS.pop(scheme, None)


def _client(url: str) -> SchemeClient:
    scheme = urlparse(url).scheme
    if scheme not in _CLIENTS:
        if scheme not in _CLIENT_FACTORIES:
            raise NotImplementedError(f"no client registered for '{scheme}://' URLs")
        _CLIENTS[scheme] = _CLIENT_FACTORIES[scheme]()
    return _CLIENTS[scheme]


class _HttpClient(SchemeClient):
    def _requests(self):
        import requests

        return requests

    def exists(self, url: str) -> bool:
        return self._requests().head(url, allow_redirects=True, timeout=30).status_code == 200

    def size(self, url: str) -> int:
        r = self._requests().head(url, allow_redirects=True, timeout=30)
        if r.status_code != 200:
            raise FileNotFoundError(url)
        return int(r.headers["content-length"])

    def read_range(self, url: str, start: int, length: int) -> bytes:
        r = self._requests().get(url, headers={"Range": f"bytes={start}-{start + length - 1}"}, timeout=60)
        if r.status_code == 404:
            raise FileNotFoundError(url)
        if r.status_code == 416:
            raise OLMoInvalidRangeRequestError(f"bad range {start}+{length} for {url}")
        if r.status_code not in (200, 206):
            raise OLMoNetworkError(f"GET {url} -> {r.status_code}")
        return r.content if r.status_code == 206 else r.content[start : start + length]


class _S3Client(SchemeClient):
    """S3-compatible stores (``s3``, ``r2``, ``weka``); endpoint/profile from ``<SCHEME>_ENDPOINT_URL`` / ``<SCHEME>_PROFILE``."""

    def __init__(self, scheme: str):
        try:
            import boto3  # type: ignore
            from botocore.config import Config as BotoConfig  # type: ignore
        except ImportError as e:
            raise OLMoEnvironmentError(f"'{scheme}://' URLs need boto3, which is not installed") from e
        self.scheme = scheme
        endpoint = os.environ.get(f"{scheme.upper()}_ENDPOINT_URL")
        profile = os.environ.get(f"{scheme.upper()}_PROFILE")
        session = boto3.Session(profile_name=profile) if profile else boto3.Session()
        self.client = session.client("s3", endpoint_url=endpoint, config=BotoConfig(retries={"max_attempts": 10, "mode": "standard"}))

    @staticmethod
    def _split(url: str) -> Tuple[str, str]:
        p = urlparse(url)
        return p.netloc, p.path.lstrip("/")

    def exists(self, url: str) -> bool:
        try:
            self.size(url)
            return True
        except FileNotFoundError:
            return False

    def size(self, url: str) -> int:
        b, k = self._split(url)
        try:
            return int(self.client.head_object(Bucket=b, Key=k)["ContentLength"])
        except Exception as e:  # botocore ClientError 404
            if "404" in str(e) or "Not Found" in str(e):
                raise FileNotFoundError(url) from e
            raise OLMoNetworkError(str(e)) from e

    def read_range(self, url: str, start: int, length: int) -> bytes:
        b, k = self._split(url)
        try:
            return self.client.get_object(Bucket=b, Key=k, Range=f"bytes={start}-{start + length - 1}")["Body"].read()
        except Exception as e:
            if "NoSuchKey" in str(e) or "404" in str(e):
                raise FileNotFoundError(url) from e
            raise OLMoNetworkError(str(e)) from e

    def upload(self, source: Path, url: str, overwrite: bool) -> None:
        if not overwrite and self.exists(url):
            raise FileExistsError(url)
        b, k = self._split(url)
        self.client.upload_file(str(source), b, k)

    def delete(self, url: str) -> None:
        b, k = self._split(url)
        self.client.delete_object(Bucket=b, Key=k)

    def list(self, url: str, recurse: bool) -> List[str]:
        b, k = self._split(url)
        prefix = k.rstrip("/") + "/"
        out: List[str] = []
        kwargs: Dict[str, Any] = dict(Bucket=b, Prefix=prefix)
        if not recurse:
            kwargs["Delimiter"] = "/"
        for page in self.client.get_paginator("list_objects_v2").paginate(**kwargs):
            out += [f"{self.scheme}://{b}/{o['Key']}" for o in page.get("Contents", [])]
            out += [f"{self.scheme}://{b}/{p['Prefix'].rstrip('/')}" for p in page.get("CommonPrefixes", [])]
        return out


class _GCSClient(SchemeClient):
    scheme = "gs"

    def __init__(self):
        try:
            from google.cloud import storage  # type: ignore
        except ImportError as e:
            raise OLMoEnvironmentError("'gs://' URLs need google-cloud-storage, which is not installed") from e
        self.client = storage.Client()

    def _blob(self, url: str):
        p = urlparse(url)
        return self.client.bucket(p.netloc).blob(p.path.lstrip("/"))

    def exists(self, url: str) -> bool:
        return self._blob(url).exists()

    def size(self, url: str) -> int:
        blob = self._blob(url)
        blob.reload()
        return int(blob.size)

    def read_range(self, url: str, start: int, length: int) -> bytes:
        return self._blob(url).download_as_bytes(start=start, end=start + length - 1)

    def upload(self, source: Path, url: str, overwrite: bool) -> None:
        blob = self._blob(url)
        if not overwrite and blob.exists():
            raise FileExistsError(url)
        blob.upload_from_filename(str(source))

    def delete(self, url: str) -> None:
        self._blob(url).delete()

    def list(self, url: str, recurse: bool) -> List[str]:
        p = urlparse(url)
        prefix = p.path.lstrip("/").rstrip("/") + "/"
        it = self.client.list_blobs(p.netloc, prefix=prefix, delimiter=None if recurse else "/")
        out = [f"gs://{p.netloc}/{b.name}" for b in it]
        out += [f"gs://{p.netloc}/{pre.rstrip('/')}" for pre in getattr(it, "prefixes", [])]
        return out


register_scheme_client("http", _HttpClient)
register_scheme_client("https", _HttpClient)
for _s in ("s3", "r2", "weka"):
    register_scheme_client(_s, functools.partial(_S3Client, _s))
register_scheme_client("gs", _GCSClient)


def init_client(remote_path: str) -> None:
    """Create the client for ``remote_path``'s scheme up front (so worker threads do not race)."""
    if is_url(remote_path) and urlparse(remote_path).scheme != "file":
        _client(remote_path)


def add_cached_path_clients() -> None:
    """Kept for API parity; scheme clients register themselves on import."""


# ----------------------------------------------------------------------------------------------
# file operations
# ----------------------------------------------------------------------------------------------


def resource_path(folder: PathOrStr, fname: str, local_cache: Optional[PathOrStr] = None) -> Path:
    """Local path of ``folder/fname``, downloading it first when ``folder`` is a URL."""
    folder = normalize_path(folder)
    if local_cache is not None and (Path(local_cache) / fname).is_file():
        return Path(local_cache) / fname
    if not is_url(folder):
        return Path(folder) / fname
    url = f"{folder}/{fname}"
    cache_dir = Path(local_cache or os.environ.get("OLMO_CACHE_DIR", Path.home() / ".cache" / "olmo_core_b200"))
    target = cache_dir / re.sub(r"[^A-Za-z0-9._-]", "_", url)
    if not target.is_file():
        target.parent.mkdir(parents=True, exist_ok=True)
        tmp = target.with_suffix(target.suffix + f".tmp{os.getpid()}")
        tmp.write_bytes(read_bytes(url))
        tmp.replace(target)
    return target


def file_exists(path: PathOrStr) -> bool:
    p = normalize_path(path)
    if is_url(p):
        return _client(p).exists(p)
    return Path(p).exists()


def dir_is_empty(dir: PathOrStr) -> bool:
    d = normalize_path(dir)
    if is_url(d):
        return len(_client(d).list(d, False)) == 0
    p = Path(d)
    if not p.is_dir():
        return True
    return next(p.iterdir(), None) is None


def get_file_size(path: PathOrStr) -> int:
    p = normalize_path(path)
    if is_url(p):
        return _client(p).size(p)
    return os.stat(p).st_size


@retriable()
def get_bytes_range(path: PathOrStr, bytes_start: int, num_bytes: int) -> bytes:
    """Read ``num_bytes`` starting at ``bytes_start``."""
    p = normalize_path(path)
    if is_url(p):
        return _client(p).read_range(p, bytes_start, num_bytes)
    with open(p, "rb") as f:
        f.seek(bytes_start)
        return f.read(num_bytes)


def read_bytes(path: PathOrStr) -> bytes:
    p = normalize_path(path)
    if is_url(p):
        return get_bytes_range(p, 0, get_file_size(p))
    return Path(p).read_bytes()


def read_text(path: PathOrStr) -> str:
    return read_bytes(path).decode("utf-8")


def write_bytes(path: PathOrStr, data: bytes, overwrite: bool = True) -> None:
    p = normalize_path(path)
    if is_url(p):
        import tempfile

        with tempfile.NamedTemporaryFile(delete=False) as tmp:
            tmp.write(data)
        try:
            upload(tmp.name, p, save_overwrite=overwrite)
        finally:
            os.unlink(tmp.name)
        return
    target = Path(p)
    if target.exists() and not overwrite:
        raise FileExistsError(p)
    target.parent.mkdir(parents=True, exist_ok=True)
    tmp_path = target.with_name(target.name + f".tmp{os.getpid()}")
    with open(tmp_path, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    tmp_path.replace(target)


def write_text(path: PathOrStr, text: str, overwrite: bool = True) -> None:
    write_bytes(path, text.encode("utf-8"), overwrite)


@retriable()
def upload(source: PathOrStr, target: str, save_overwrite: bool = False, quiet: bool = False) -> None:
    """Upload local ``source`` to URL ``target``."""
    t = normalize_path(target)
    if not is_url(t):
        copy_file(source, t, save_overwrite=save_overwrite, quiet=quiet)
        return
    if not quiet:
        log.info(f"Uploading {source} to {t}...")
    _client(t).upload(Path(source), t, save_overwrite)


def copy_file(source: PathOrStr, target: PathOrStr, save_overwrite: bool = False, quiet: bool = False) -> None:
    s, t = normalize_path(source), normalize_path(target)
    if is_url(t):
        if is_url(s):
            write_bytes(t, read_bytes(s), overwrite=save_overwrite)
        else:
            upload(s, t, save_overwrite=save_overwrite, quiet=quiet)
        return
    tp = Path(t)
    if tp.exists() and not save_overwrite:
        raise FileExistsError(t)
    tp.parent.mkdir(parents=True, exist_ok=True)
    if is_url(s):
        write_bytes(t, read_bytes(s))
    else:
        shutil.copyfile(s, t)


def copy_dir(source: PathOrStr, target: PathOrStr, save_overwrite: bool = False, num_threads: Optional[int] = None,
             quiet: bool = False) -> None:
    from concurrent.futures import ThreadPoolExecutor

    s = normalize_path(source)
    files = list(list_directory(s, recurse=True, include_dirs=False))
    if not quiet:
        log.info(f"Copying {len(files):,d} files from {s} to {target}...")
    with ThreadPoolExecutor(max_workers=num_threads or 8) as pool:
        futs = []
        for f in files:
            rel = str(f)[len(s):].lstrip("/")
            futs.append(pool.submit(copy_file, f, join_path(target, rel), save_overwrite, True))
        for fu in futs:
            fu.result()


def remove_file(path: PathOrStr) -> None:
    p = normalize_path(path)
    if is_url(p):
        _client(p).delete(p)
    else:
        Path(p).unlink(missing_ok=True)


def clear_directory(dir: PathOrStr, force: bool = False) -> None:
    """Delete ``dir`` and everything under it."""
    d = normalize_path(dir)
    if is_url(d):
        for f in _client(d).list(d, True):
            _client(d).delete(f)
        return
    if Path(d).exists():
        shutil.rmtree(d, ignore_errors=True)


def list_directory(
    dir: PathOrStr, recurse: bool = False, include_files: bool = True, include_dirs: bool = True
) -> Generator[str, None, None]:
    d = normalize_path(dir)
    if is_url(d):
        for f in _client(d).list(d, recurse):
            yield f
        return
    root = Path(d)
    if not root.is_dir():
        return
    for p in sorted(root.iterdir()):
        if p.is_dir():
            if include_dirs:
                yield str(p)
            if recurse:
                yield from list_directory(p, recurse, include_files, include_dirs)
        elif include_files:
            yield str(p)


def glob_directory(pattern: str) -> Generator[str, None, None]:
    import fnmatch
    import glob as _glob

    if not is_url(pattern):
        yield from sorted(_glob.glob(pattern, recursive=True))
        return
    base = pattern.split("*", 1)[0].rsplit("/", 1)[0]
    for f in list_directory(base, recurse=True, include_dirs=False):
        if fnmatch.fnmatch(f, pattern):
            yield f


def serialize_to_tensor(x: Any) -> torch.Tensor:
    """Pickle an object into a ``uint8`` tensor (for sending through tensor collectives)."""
    return torch.frombuffer(bytearray(pickle.dumps(x)), dtype=torch.uint8)


def deserialize_from_tensor(data: torch.Tensor) -> Any:
    return pickle.loads(bytearray(data.cpu().numpy().tobytes()))


def deterministic_glob_directory(pattern: str) -> List[str]:
    """:func:`glob_directory` as a sorted list, so that every rank and every run sees the same order."""
    return sorted(glob_directory(pattern))
