"""
Storage layer of the sharded checkpoint format: a ``torch.distributed.checkpoint`` ``StorageWriter`` /
``StorageReader`` pair that works on local paths and URLs
(on-disk format of src/olmo_core/distributed/checkpoint/filesystem.py:56-480):

* every rank writes files ``__{rank}_{i}.distcp``; each file is a concatenation of ``torch.save`` blobs, one
  per tensor shard (or pickled object), written to a temporary name, fsync'ed and renamed (or uploaded);
* the coordinator pickles the ``Metadata`` -- with ``storage_data`` mapping each ``MetadataIndex`` to a
  ``_StorageInfo(relative_path, offset, length)`` -- into ``.metadata``;
* the reader fetches exactly the byte range of each requested entry and narrows it to the wanted shard.

``_StorageInfo`` pickles under the module path ``olmo_core.distributed.checkpoint.filesystem`` so that
checkpoints are interchangeable with the reference implementation in both directions.
"""

from __future__ import annotations

import io
import logging
import os
import pickle
import tempfile
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed.checkpoint as dist_cp
from torch.distributed.checkpoint.metadata import Metadata, MetadataIndex, StorageMeta
from torch.distributed.checkpoint.planner import (
    LoadItemType,
    LoadPlan,
    LoadPlanner,
    ReadItem,
    SavePlan,
    SavePlanner,
    WriteItem,
    WriteItemType,
)
from torch.distributed.checkpoint.storage import WriteResult
from torch.futures import Future

from ...aliases import PathOrStr
from ...exceptions import OLMoCheckpointError
from ...io import file_exists, get_bytes_range, init_client, is_url, join_path, normalize_path, read_bytes, upload
from ...utils import generate_uuid, get_default_thread_count, get_element_size
from ..utils import do_n_at_a_time

log = logging.getLogger(__name__)

__all__ = ["RemoteFileSystemWriter", "RemoteFileSystemReader"]

_REFERENCE_MODULE = "olmo_core.distributed.checkpoint.filesystem"


@dataclass
class _StorageInfo:
    """Where one checkpoint entry lives: file (relative to the checkpoint dir), byte offset and length."""

    relative_path: str
    offset: int
    length: int


@dataclass
class _StoragePrefix:
    prefix: str


_StorageInfo.__module__ = _REFERENCE_MODULE
_StoragePrefix.__module__ = _REFERENCE_MODULE


def _item_bytes(item: WriteItem) -> int:
    if item.tensor_data is None:
        return 0
    n = 1
    for s in item.tensor_data.size:
        n *= s
    return n * get_element_size(item.tensor_data.properties.dtype)


def _balance(bins: int, items: List[WriteItem]) -> List[List[WriteItem]]:
    """Greedy largest-first packing of write items into ``bins`` files of similar size."""
    if bins <= 1:
        return [items]
    buckets: List[List[WriteItem]] = [[] for _ in range(bins)]
    sizes = [0] * bins
    blobs = [w for w in items if w.type == WriteItemType.BYTE_IO]
    tensors = sorted((w for w in items if w.type != WriteItemType.BYTE_IO), key=_item_bytes, reverse=True)
    for i, w in enumerate(blobs):
        buckets[i % bins].append(w)
    for w in tensors:
        j = sizes.index(min(sizes))
        buckets[j].append(w)
        sizes[j] += _item_bytes(w)
    return [b for b in buckets if b]


def _write_file(items: List[WriteItem], planner: SavePlanner, rel_name: str, root: str, overwrite: bool) -> List[WriteResult]:
    """Serialise ``items`` back to back into one file and place it at ``root/rel_name``."""
    results: List[WriteResult] = []
    target = f"{root}/{rel_name}"
    tmp = Path(tempfile.mkdtemp()) / rel_name if is_url(root) else Path(f"{target}-{generate_uuid()}.tmp")
    tmp.parent.mkdir(parents=True, exist_ok=True)
    with open(tmp, "wb") as f:
        for item in items:
            offset = f.tell()
            data = planner.resolve_data(item)
            if item.type == WriteItemType.BYTE_IO:
                assert isinstance(data, io.BytesIO)
                f.write(data.getbuffer())
            else:
                assert isinstance(data, torch.Tensor)
                t = data.detach()
                if t.device.type != "cpu":
                    t = t.cpu()
                if t.untyped_storage().size() != t.numel() * t.element_size():
                    t = t.clone()  # do not serialise the whole backing buffer of a view
                torch.save(t, f)
            results.append(WriteResult(index=item.index, size_in_bytes=f.tell() - offset,
                                       storage_data=_StorageInfo(rel_name, offset, f.tell() - offset)))
        f.flush()
        os.fsync(f.fileno())
    if is_url(root):
        try:
            upload(tmp, target, save_overwrite=overwrite)
        finally:
            tmp.unlink(missing_ok=True)
    else:
        if Path(target).exists() and not overwrite:
            tmp.unlink(missing_ok=True)
            raise FileExistsError(target)
        tmp.replace(target)
    return results


class RemoteFileSystemWriter(dist_cp.StorageWriter):
    def __init__(self, path: PathOrStr, thread_count: Optional[int] = None, save_overwrite: bool = False,
                 process_group=None, throttle_uploads: bool = False, process_count: Optional[int] = None):
        super().__init__()
        if thread_count is not None and thread_count <= 0:
            raise ValueError("thread count must be at least 1")
        self.path = normalize_path(path)
        # Serialisation here is a device->host copy plus a file write, both of which release the interpreter lock,
        # so a request for worker processes is served by as many writer threads.
        self.process_count = process_count
        self.thread_count = thread_count or process_count or get_default_thread_count()
        self.save_overwrite = save_overwrite
        self.process_group = process_group
        self.throttle_uploads = throttle_uploads
        self.save_id = generate_uuid()

    def reset(self, checkpoint_id: Union[str, os.PathLike, None] = None) -> None:
        if checkpoint_id:
            self.path = normalize_path(checkpoint_id)
        self.save_id = generate_uuid()

    @classmethod
    def validate_checkpoint_id(cls, checkpoint_id: Union[str, os.PathLike]) -> bool:
        return True

    def set_up_storage_writer(self, is_coordinator: bool, *args, **kwargs) -> None:
        if is_url(self.path):
            init_client(self.path)
        else:
            Path(self.path).mkdir(parents=True, exist_ok=True)

    def prepare_local_plan(self, plan: SavePlan) -> SavePlan:
        return plan

    def prepare_global_plan(self, plans: List[SavePlan]) -> List[SavePlan]:
        import dataclasses

        return [dataclasses.replace(p, storage_data=_StoragePrefix(f"__{i}_")) for i, p in enumerate(plans)]

    def write_data(self, plan: SavePlan, planner: SavePlanner) -> Future:
        prefix: _StoragePrefix = plan.storage_data
        groups = _balance(self.thread_count, list(plan.items))

        def run() -> List[WriteResult]:
            out: List[WriteResult] = []
            with ThreadPoolExecutor(max_workers=max(1, len(groups))) as pool:
                futs = [pool.submit(_write_file, g, planner, f"{prefix.prefix}{i}.distcp", self.path, self.save_overwrite)
                        for i, g in enumerate(groups)]
                for fu in futs:
                    out.extend(fu.result())
            return out

        results = do_n_at_a_time(run, n=8, process_group=self.process_group) if (self.throttle_uploads and is_url(self.path)) else run()
        fut: Future = Future()
        fut.set_result(results)
        return fut

    def finish(self, metadata: Metadata, results: List[List[WriteResult]]) -> None:
        metadata.storage_data = {r.index: r.storage_data for rank_results in results for r in rank_results}
        metadata.storage_meta = self.storage_meta()
        blob = pickle.dumps(metadata)
        target = self.metadata_path
        if is_url(self.path):
            with tempfile.NamedTemporaryFile(delete=False) as tmp:
                tmp.write(blob)
            try:
                upload(tmp.name, target, save_overwrite=self.save_overwrite)
            finally:
                os.unlink(tmp.name)
        else:
            tmp_path = Path(f"{target}.tmp")
            with open(tmp_path, "wb") as f:
                f.write(blob)
                f.flush()
                os.fsync(f.fileno())
            tmp_path.replace(target)

    def storage_meta(self) -> Optional[StorageMeta]:
        return StorageMeta(checkpoint_id=self.path, save_id=self.save_id)

    @property
    def metadata_path(self) -> str:
        return f"{self.path}/.metadata"

    @property
    def checkpoint_id(self) -> str:
        """Where the checkpoint is being written."""
        return self.path


class RemoteFileSystemReader(dist_cp.StorageReader):
    def __init__(self, path: PathOrStr, *, thread_count: Optional[int] = None, pre_download: bool = False,
                 work_dir: Optional[PathOrStr] = None):
        super().__init__()
        self.path = normalize_path(path)
        self.thread_count = thread_count or get_default_thread_count()
        self.pre_download = pre_download
        self.work_dir = work_dir
        self.storage_data: Dict[MetadataIndex, _StorageInfo] = {}
        self._metadata: Optional[Metadata] = None
        self._local_cache: Dict[str, str] = {}

    def reset(self, checkpoint_id: Union[str, os.PathLike, None] = None) -> None:
        if checkpoint_id:
            self.path = normalize_path(checkpoint_id)
        self._metadata = None
        self.storage_data = {}

    @property
    def checkpoint_id(self) -> str:
        return self.path

    @classmethod
    def validate_checkpoint_id(cls, checkpoint_id: Union[str, os.PathLike]) -> bool:
        return True

    def _read_entry(self, info: _StorageInfo) -> bytes:
        src = f"{self.path}/{info.relative_path}"
        if self.pre_download and is_url(self.path):
            local = self._local_cache.get(info.relative_path)
            if local is None:
                d = Path(self.work_dir or tempfile.mkdtemp())
                d.mkdir(parents=True, exist_ok=True)
                local = str(d / info.relative_path)
                Path(local).write_bytes(read_bytes(src))
                self._local_cache[info.relative_path] = local
            src = local
        return get_bytes_range(src, info.offset, info.length)

    def _load_item(self, item: ReadItem, planner: LoadPlanner) -> None:
        info = self.storage_data[item.storage_index]
        raw = self._read_entry(info)
        if len(raw) != info.length:
            raise OLMoCheckpointError(
                f"'{self.path}/{info.relative_path}' is truncated: entry '{item.storage_index.fqn}' needs bytes "
                f"[{info.offset}, {info.offset + info.length}) but only {len(raw)} could be read")
        if item.type == LoadItemType.BYTE_IO:
            planner.load_bytes(item, io.BytesIO(raw))
            return
        try:
            tensor = torch.load(io.BytesIO(raw), map_location="cpu", weights_only=False)
        except Exception as e:
            raise OLMoCheckpointError(f"'{self.path}/{info.relative_path}' is damaged: entry '{item.storage_index.fqn}' "
                                      f"cannot be decoded ({type(e).__name__}: {e})") from e
        for dim, (off, length) in enumerate(zip(item.storage_offsets, item.lengths)):
            tensor = torch.narrow(tensor, dim, off, length)
        target = planner.resolve_tensor(item).detach()
        if target.size() != tensor.size():
            raise OLMoCheckpointError(f"{item.storage_index}: shape mismatch, {tuple(target.size())} vs {tuple(tensor.size())}")
        target.copy_(tensor)
        planner.commit_tensor(item, target)

    def read_data(self, plan: LoadPlan, planner: LoadPlanner) -> Future:
        with ThreadPoolExecutor(max_workers=self.thread_count) as pool:
            for fu in [pool.submit(self._load_item, it, planner) for it in plan.items]:
                fu.result()
        fut: Future = Future()
        fut.set_result(None)
        return fut

    def read_metadata(self) -> Metadata:
        if self._metadata is None:
            try:
                self._metadata = _CompatUnpickler(io.BytesIO(read_bytes(f"{self.path}/.metadata"))).load()
            except FileNotFoundError as e:
                raise FileNotFoundError(f"'{self.path}' is not a distributed checkpoint folder (no .metadata)") from e
            if getattr(self._metadata, "storage_meta", None) is None:
                self._metadata.storage_meta = StorageMeta()
        return self._metadata

    def set_up_storage_reader(self, metadata: Metadata, is_coordinator: bool, *args, **kwargs) -> None:
        self.storage_data = metadata.storage_data

    def prepare_local_plan(self, plan: LoadPlan) -> LoadPlan:
        return plan

    def prepare_global_plan(self, global_plan: List[LoadPlan]) -> List[LoadPlan]:
        return global_plan


class _CompatUnpickler(pickle.Unpickler):
    """Resolves the storage-info classes whichever implementation wrote the checkpoint."""

    def find_class(self, module: str, name: str):
        if name in ("_StorageInfo", "_StoragePrefix") and module.endswith("distributed.checkpoint.filesystem"):
            return {"_StorageInfo": _StorageInfo, "_StoragePrefix": _StoragePrefix}[name]
        return super().find_class(module, name)
