"""
Reading sharded checkpoints without a model: full (unsharded) tensors by key, whole-checkpoint unsharding to
``torch.save`` / safetensors files, and the checkpoint's metadata
(behaviour of src/olmo_core/distributed/checkpoint/__init__.py:396-767).

Unsharded layouts written by :func:`unshard_checkpoint` under ``target_dir``:

=====================  ==========================================================================
strategy               files
=====================  ==========================================================================
``one_file``           ``model.pt`` (and ``optim.pt``)
``one_file_per_tensor````model/<flat-key-with-dashes>.pt``
``chunks``             ``model/chunk-00000.pt`` ... each at most about ``chunk_size_bytes`` large
=====================  ==========================================================================
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Generator, Iterable, List, Optional, Tuple

import torch
import torch.distributed.checkpoint as dist_cp
from torch.distributed.checkpoint.metadata import BytesStorageMetadata, Metadata, TensorStorageMetadata

from ...aliases import PathOrStr
from ...config import StrEnum
from ...io import normalize_path
from ...utils import gc_cuda, get_element_size
from .filesystem import RemoteFileSystemReader

log = logging.getLogger(__name__)

__all__ = ["UnshardStrategyType", "UnshardStrategy", "unshard_checkpoint", "load_keys", "get_checkpoint_metadata",
           "load_unsharded_keys"]


class UnshardStrategyType(StrEnum):
    one_file = "one_file"
    """Model state in one file, optimizer state in another. Needs host memory for the whole state."""

    one_file_per_tensor = "one_file_per_tensor"
    """One file per tensor (model state only); host memory for one tensor at a time."""

    chunks = "chunks"
    """Several tensors per file, up to about :data:`UnshardStrategy.chunk_size_bytes` each."""


@dataclass
class UnshardStrategy:
    name: UnshardStrategyType = UnshardStrategyType.one_file
    chunk_size_bytes: Optional[int] = None

    def __post_init__(self):
        if self.name == UnshardStrategyType.chunks and self.chunk_size_bytes is None:
            raise ValueError("'chunk_size_bytes' is required for the 'chunks' strategy")
        if self.name != UnshardStrategyType.chunks and self.chunk_size_bytes is not None:
            raise ValueError("'chunk_size_bytes' is only valid for the 'chunks' strategy")

    @classmethod
    def one_file(cls) -> "UnshardStrategy":
        return cls(name=UnshardStrategyType.one_file)

    @classmethod
    def one_file_per_tensor(cls) -> "UnshardStrategy":
        return cls(name=UnshardStrategyType.one_file_per_tensor)

    @classmethod
    def chunks(cls, chunk_size_in_bytes: int) -> "UnshardStrategy":
        return cls(name=UnshardStrategyType.chunks, chunk_size_bytes=chunk_size_in_bytes)


def get_checkpoint_metadata(dir: PathOrStr) -> Metadata:
    """The ``torch.distributed.checkpoint`` metadata (keys, shapes, dtypes, chunking) of the checkpoint at ``dir``."""
    return RemoteFileSystemReader(normalize_path(dir)).read_metadata()


def _entry_bytes(meta: Any) -> int:
    if isinstance(meta, TensorStorageMetadata):
        n = 1
        for s in meta.size:
            n *= s
        return n * get_element_size(meta.properties.dtype)
    return 0


def _matching_keys(metadata: Metadata, keys: Iterable[str]) -> List[str]:
    """Metadata keys equal to, or nested under, any of ``keys`` -- in metadata order."""
    wanted = list(keys)
    return [k for k in metadata.state_dict_metadata
            if any(k == w or k.startswith(w + ".") for w in wanted)]


def _nest(flat: Dict[str, Any], metadata: Metadata) -> Dict[str, Any]:
    """Rebuild the nesting that the state dict had when it was saved (recorded in the planner data)."""
    paths = getattr(metadata, "planner_data", None) or {}
    out: Dict[str, Any] = {}
    for key, value in flat.items():
        path = paths.get(key)
        parts = [str(p) for p in path] if path else key.split(".", 1) if "." in key else [key]
        node = out
        for part in parts[:-1]:
            node = node.setdefault(part, {})
        node[parts[-1]] = value
    return out


def load_unsharded_keys(dir: PathOrStr, keys: Iterable[str], *, pre_download: bool = False,
                        work_dir: Optional[PathOrStr] = None, nested: bool = True) -> Dict[str, Any]:
    """
    Load the full value of every checkpoint entry equal to or nested under one of ``keys`` into host memory.
    Runs in the calling process only (no collective), whatever the world size that wrote the checkpoint.
    """
    dir = normalize_path(dir)
    reader = RemoteFileSystemReader(dir, pre_download=pre_download, work_dir=work_dir)
    metadata = reader.read_metadata()
    flat: Dict[str, Any] = {}
    for k in _matching_keys(metadata, keys):
        meta = metadata.state_dict_metadata[k]
        if isinstance(meta, TensorStorageMetadata):
            flat[k] = torch.empty(tuple(meta.size), dtype=meta.properties.dtype, device="cpu")
        elif isinstance(meta, BytesStorageMetadata):
            flat[k] = None
    if not flat:
        return {}
    dist_cp.state_dict_loader.load(flat, checkpoint_id=dir, storage_reader=reader, no_dist=True)
    return _nest(flat, metadata) if nested else flat


def load_keys(dir: PathOrStr, keys: Iterable[str], *, pre_download: bool = False,
              work_dir: Optional[PathOrStr] = None) -> Generator[Any, None, None]:
    """Yield the full value of each of ``keys`` (exact flat keys such as ``model.embeddings.weight``), in order."""
    keys = list(keys)
    flat = load_unsharded_keys(dir, keys, pre_download=pre_download, work_dir=work_dir, nested=False)
    for k in keys:
        if k not in flat:
            raise KeyError(f"'{k}' not found in checkpoint '{dir}'")
        yield flat[k]


def unshard_checkpoint(
    dir: PathOrStr,
    target_dir: PathOrStr,
    *,
    optim: Optional[bool] = None,
    save_overwrite: bool = False,
    use_safetensors: bool = False,
    unshard_strategy: Optional[UnshardStrategy] = None,
    pre_download: bool = False,
    work_dir: Optional[PathOrStr] = None,
    quiet: bool = False,
) -> Tuple[Path, Optional[Path]]:
    """
    Convert a sharded checkpoint into plain files loadable with ``torch.load`` (or safetensors). Returns the
    model path and the optimizer path (files or directories depending on the strategy). Call it from a single
    process.
    """
    strategy = unshard_strategy or UnshardStrategy.one_file()
    if optim is None:
        optim = not use_safetensors and strategy.name == UnshardStrategyType.one_file
    elif optim and use_safetensors:
        raise NotImplementedError("`optim=True` is incompatible with `use_safetensors=True`")
    elif optim and strategy.name == UnshardStrategyType.one_file_per_tensor:
        raise NotImplementedError("`optim=True` is incompatible with the 'one_file_per_tensor' strategy")
    dir = normalize_path(dir)
    target = Path(normalize_path(target_dir))
    if "://" in str(target_dir):
        raise NotImplementedError("'target_dir' must be a local directory")
    target.mkdir(parents=True, exist_ok=True)
    ext = "safetensors" if use_safetensors else "pt"
    metadata = get_checkpoint_metadata(dir)

    def write(state: Dict[str, Any], path: Path) -> None:
        if path.is_file() and not save_overwrite:
            raise FileExistsError(f"'{path}' already exists, use `save_overwrite=True` to overwrite it")
        path.parent.mkdir(parents=True, exist_ok=True)
        if use_safetensors:
            from safetensors.torch import save_file

            save_file(state, str(path))
        else:
            torch.save(state, path)

    def plan(prefix: str) -> Tuple[Path, List[Tuple[Path, List[str]]]]:
        entries = [k for k in metadata.state_dict_metadata if k.startswith(prefix + ".")]
        if strategy.name == UnshardStrategyType.one_file:
            path = target / f"{prefix}.{ext}"
            return path, [(path, [prefix])]
        root = target / prefix
        if strategy.name == UnshardStrategyType.one_file_per_tensor:
            return root, [(root / f"{k.replace('.', '-')}.{ext}", [k]) for k in entries]
        assert strategy.chunk_size_bytes is not None
        groups: List[Tuple[Path, List[str]]] = []
        cur: List[str] = []
        cur_bytes = 0
        for k in entries:
            size = _entry_bytes(metadata.state_dict_metadata[k])
            if cur and cur_bytes + size > strategy.chunk_size_bytes:
                groups.append((root / f"chunk-{len(groups):05d}.{ext}", cur))
                cur, cur_bytes = [], 0
            cur.append(k)
            cur_bytes += size
        if cur:
            groups.append((root / f"chunk-{len(groups):05d}.{ext}", cur))
        return root, groups

    def run(prefix: str) -> Path:
        path, groups = plan(prefix)
        for i, (file, keys) in enumerate(groups):
            if not quiet:
                log.info(f"Unsharding {prefix} ({i + 1}/{len(groups)}) -> {file}")
            state = load_unsharded_keys(dir, keys, pre_download=pre_download, work_dir=work_dir)
            if not state or prefix not in state:
                raise RuntimeError(f"missing keys '{keys}' in checkpoint")
            write(state[prefix], file)
            del state
            gc_cuda()
        return path

    model_path = run("model")
    optim_path = run("optim") if optim else None
    return model_path, optim_path
