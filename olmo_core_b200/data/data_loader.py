"""
Data loaders for the trainer (interface and data order of src/olmo_core/data/data_loader.py:54-1167).

A loader yields, on every data-parallel rank, that rank's slice of each global batch; it is resumable (``state_dict``)
and reproducible: the order of an epoch is a seeded permutation of the instance indices stored in (or memory-mapped
from) the work directory, so it does not depend on the number of ranks, threads or the batch size.

Loading is *batch addressed*: batch ``k`` of an epoch is a pure function of ``k`` (``loader[k]``). Iteration keeps a
window of the next batches in flight on a thread pool -- token windows are read with ``pread``-style ranged reads that
release the GIL -- and, for CUDA targets, collates into pinned host memory so that the trainer's host-to-device copy
is asynchronous. No worker processes are forked; ``num_workers`` only scales the depth of the prefetch window.
"""

from __future__ import annotations

import logging
from abc import ABC, abstractmethod
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Generic, Iterable, Iterator, List, Optional, Tuple, TypeVar

import numpy as np
import torch
import torch.distributed as dist

from ..aliases import PathOrStr
from ..config import Config, Registrable
from ..distributed.parallel import get_dp_process_group
from ..distributed.utils import barrier, get_fs_local_rank, get_rank, get_world_size
from ..exceptions import OLMoConfigurationError
from ..io import is_url, normalize_path
from ..utils import get_default_device
from .collator import DataCollator
from .numpy_dataset import NumpyDatasetBase, NumpyFSLDatasetBase, NumpyVSLDataset
from .utils import get_rng, load_array_slice, write_array_to_disk

log = logging.getLogger(__name__)

__all__ = ["DataLoaderBase", "TextDataLoaderBase", "NumpyDataLoaderBase", "NumpyFSLDataLoader", "NumpyVSLDataLoader",
           "DataLoaderConfig", "NumpyDataLoaderConfig"]


class DataLoaderBase(ABC):
    """
    What the trainer needs from a data loader. ``global_batch_size`` is in whatever unit the loader counts (tokens for
    text); changing it mid-epoch rescales ``batches_processed`` so that the position in the data is kept.
    """

    def __init__(self, *, work_dir: PathOrStr, global_batch_size: int, dp_world_size: int = 1, dp_rank: int = 0,
                 fs_local_rank: Optional[int] = None):
        if is_url(work_dir):
            raise OLMoConfigurationError(f"'work_dir' should be a local path, not a URL ('{work_dir}').")
        assert dp_rank < dp_world_size
        self.work_dir = Path(normalize_path(work_dir))
        self._global_batch_size = global_batch_size
        self.dp_world_size = dp_world_size
        self.dp_rank = dp_rank
        self.fs_local_rank = fs_local_rank if fs_local_rank is not None else get_fs_local_rank()
        self.batches_processed = 0
        """Batches consumed so far in the current epoch."""
        self._epoch: Optional[int] = None

    @property
    def global_batch_size(self) -> int:
        return self._global_batch_size

    @global_batch_size.setter
    def global_batch_size(self, new: int) -> None:
        if not isinstance(new, int):
            raise TypeError(f"expected int, got {type(new)}")
        old = self._global_batch_size
        if new > old:
            if new % old != 0:
                raise RuntimeError("global batch size can only be increased by an integer factor")
            ratio = new // old
            if self.batches_processed % ratio != 0:
                raise RuntimeError(
                    f"increasing global batch size by a factor of {ratio} is only possible after a multiple of {ratio} "
                    f"batches (no data may be skipped or repeated); {self.batches_processed:d} have been processed."
                )
            self.batches_processed //= ratio
        elif new < old:
            if old % new != 0:
                raise RuntimeError("global batch size can only be decreased by an integer factor")
            self.batches_processed *= old // new
        self._global_batch_size = new

    @property
    def epoch(self) -> int:
        """The current epoch (1-based); set by :meth:`reshuffle`."""
        if self._epoch is None:
            raise RuntimeError("The data loader's epoch has not been set yet, did you forget to call 'reshuffle()'?")
        return self._epoch

    @property
    @abstractmethod
    def total_batches(self) -> Optional[int]:
        """Batches in the current epoch, if known."""
        raise NotImplementedError

    def batches_in_epoch(self, epoch: int) -> Optional[int]:
        del epoch
        return self.total_batches

    def __len__(self) -> int:
        if self.total_batches is None:
            raise TypeError(f"total length (number of batches) is unknown for {self.__class__.__name__}")
        return self.total_batches

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        for batch in self._iter_batches():
            self.batches_processed += 1
            yield batch

    def __getitem__(self, index: int) -> Dict[str, Any]:
        raise TypeError(f"__getitem__ is not implemented for {self.__class__.__name__}")

    @property
    def rank_batch_size(self) -> int:
        return self.global_batch_size // self.dp_world_size

    @abstractmethod
    def state_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        raise NotImplementedError

    @abstractmethod
    def reshuffle(self, epoch: Optional[int] = None, **kwargs) -> None:
        """Prepare the order of ``epoch`` (default: the next one). Call before every epoch, also after a restore."""
        raise NotImplementedError

    @abstractmethod
    def _iter_batches(self) -> Iterable[Dict[str, Any]]:
        """This rank's slices of the remaining batches of the epoch, each exactly ``rank_batch_size`` large."""
        raise NotImplementedError

    def reset(self) -> None:
        """End-of-epoch bookkeeping."""
        self.batches_processed = 0

    @abstractmethod
    def get_mock_batch(self) -> Dict[str, Any]:
        """A batch of the right shape with arbitrary content, for the trainer's dry run."""
        raise NotImplementedError

    def global_num_tokens_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        del batch
        return None


class TextDataLoaderBase(DataLoaderBase):
    """Loaders whose batches hold ``input_ids``; batch sizes are in tokens."""

    def __init__(self, *, collator: DataCollator, work_dir: PathOrStr, global_batch_size: int, dp_world_size: int = 1,
                 dp_rank: int = 0, fs_local_rank: Optional[int] = None):
        super().__init__(work_dir=work_dir, global_batch_size=global_batch_size, dp_world_size=dp_world_size,
                         dp_rank=dp_rank, fs_local_rank=fs_local_rank)
        self.collator = collator
        self.tokens_processed: int = 0
        """Tokens (over all ranks) consumed so far in the current epoch."""

    @property
    def worker_info(self):
        """The ``torch.utils.data`` worker this code runs in, or ``None`` in the main process."""
        return torch.utils.data.get_worker_info()

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        for batch in super().__iter__():
            n = batch["input_ids"].numel()
            if n != self.rank_batch_size:
                raise RuntimeError(
                    f"Expected batch size of {self.rank_batch_size:,d} tokens on rank {self.dp_rank}, got input IDs with "
                    f"shape {tuple(batch['input_ids'].shape)} = {n:,d} tokens"
                )
            self.tokens_processed += self.global_batch_size
            yield batch

    def reset(self) -> None:
        super().reset()
        self.tokens_processed = 0

    def global_num_tokens_in_batch(self, batch: Dict[str, Any]) -> Optional[int]:
        del batch
        return self.global_batch_size


def _fname(prefix: str, **fields) -> str:
    return "_".join([prefix] + [f"{k}{fields[k]}" for k in sorted(fields) if fields[k] is not None])


class NumpyDataLoaderBase(TextDataLoaderBase):
    def __init__(self, dataset: NumpyDatasetBase, *, collator: DataCollator, global_batch_size: int, work_dir: PathOrStr,
                 seed: int = 0, shuffle: bool = True, num_threads: Optional[int] = None, num_workers: int = 0,
                 prefetch_factor: Optional[int] = None, target_device_type: str = "cpu", dp_world_size: int = 1,
                 dp_rank: int = 0, fs_local_rank: Optional[int] = None, ignore_fingerprint_mismatch: bool = False):
        super().__init__(collator=collator, work_dir=work_dir, global_batch_size=global_batch_size,
                         dp_world_size=dp_world_size, dp_rank=dp_rank, fs_local_rank=fs_local_rank)
        self.dataset = dataset
        self.seed = seed
        self.shuffle = shuffle
        self.num_threads = num_threads
        self.num_workers = num_workers
        self.prefetch_factor = prefetch_factor
        self.target_device_type = target_device_type
        self.ignore_fingerprint_mismatch = ignore_fingerprint_mismatch
        self._global_indices: Optional[np.ndarray] = None

    @classmethod
    def wrap_numpy_dataset(cls, dataset: NumpyDatasetBase, *, global_batch_size: int, collator: DataCollator,
                           work_dir: Optional[PathOrStr] = None, **kwargs) -> "NumpyDataLoaderBase":
        """The loader class that goes with ``dataset``'s class."""
        kwargs.update(global_batch_size=global_batch_size, collator=collator, work_dir=work_dir or dataset.work_dir)
        if isinstance(dataset, NumpyFSLDatasetBase):
            loader: NumpyDataLoaderBase = NumpyFSLDataLoader(dataset, **kwargs)
            if dataset.max_target_sequence_length is not None:
                # shuffle whole windows of the target length so that shorter stages see the same token order
                loader.chunk_size = dataset.max_target_sequence_length // dataset.sequence_length  # type: ignore[attr-defined]
            return loader
        if isinstance(dataset, NumpyVSLDataset):
            return NumpyVSLDataLoader(dataset, **kwargs)
        raise NotImplementedError(type(dataset))

    # -- state ----------------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return {
            "dataset_fingerprint_version": self.dataset.fingerprint_version,
            "dataset_fingerprint": self.dataset.fingerprint,
            "batches_processed": self.batches_processed,
            "tokens_processed": self.tokens_processed,
            "seed": self.seed,
            "epoch": self._epoch,
        }

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        if state_dict["dataset_fingerprint_version"] != self.dataset.fingerprint_version:
            log.warning("Dataset fingerprint version differs from the checkpoint's; the data may have changed")
        elif state_dict["dataset_fingerprint"] != self.dataset.fingerprint:
            if not self.ignore_fingerprint_mismatch:
                raise RuntimeError(
                    "Dataset fingerprint does not match the fingerprint in the checkpoint, set "
                    "ignore_fingerprint_mismatch=True to ignore this error. This will probably result in a different data order!"
                )
            log.warning("Fingerprint mismatch ignored; this will probably result in a different data order!")
        if state_dict["seed"] != self.seed:
            log.warning("Restoring data loading state with a different data seed; using the checkpoint's seed.")
            self.seed = state_dict["seed"]
        self.batches_processed = state_dict["batches_processed"]
        self.tokens_processed = state_dict["tokens_processed"]
        self._epoch = state_dict["epoch"] or self._epoch

    # -- epoch order ---------------------------------------------------------------------------------------
    @property
    @abstractmethod
    def _global_indices_file(self) -> Path:
        raise NotImplementedError

    @abstractmethod
    def _build_global_indices(self) -> np.ndarray:
        raise NotImplementedError

    @abstractmethod
    def _local_instance_indices_for_batch(self, batch_index: int) -> np.ndarray:
        """Dataset indices of this rank's instances of batch ``batch_index`` of the current epoch."""
        raise NotImplementedError

    def get_global_indices(self) -> np.ndarray:
        if self._global_indices is not None:
            return self._global_indices
        if not self._global_indices_file.is_file():
            raise RuntimeError("Missing global indices file, did you forget to call 'reshuffle()'?")
        return np.memmap(self._global_indices_file, mode="r", dtype=np.uint32)

    def build_and_save_global_indices(self, in_memory: bool = False) -> None:
        if in_memory:
            self._global_indices = self._build_global_indices()
        else:
            self._global_indices = None
            if self.fs_local_rank == 0 and not self._global_indices_file.is_file():
                log.info(f"Saving global data order indices for seed {self.seed} and epoch {self.epoch} to "
                         f"'{self._global_indices_file}'...")
                indices = self._build_global_indices()
                assert len(indices) < np.iinfo(np.uint32).max
                write_array_to_disk(indices.astype(np.uint32), self._global_indices_file)
        barrier()

    def reshuffle(self, epoch: Optional[int] = None, in_memory: bool = False, **kwargs) -> None:
        del kwargs
        if epoch is None:
            epoch = 1 if self._epoch is None else self._epoch + 1
        if epoch <= 0:
            raise ValueError(f"'epoch' must be at least 1, got {epoch}")
        self._epoch = epoch
        self.build_and_save_global_indices(in_memory=in_memory)

    # -- loading ---------------------------------------------------------------------------------------------
    def _get_dataset_item(self, idx: int) -> Dict[str, Any]:
        item = self.dataset[idx]
        return dict(**item, index=idx) if isinstance(item, dict) else {"input_ids": item, "index": idx}

    def _load_batch(self, batch_index: int, pool: Optional[ThreadPoolExecutor] = None) -> Dict[str, Any]:
        indices = [int(i) for i in self._local_instance_indices_for_batch(batch_index)]
        items = list(pool.map(self._get_dataset_item, indices)) if pool is not None else [self._get_dataset_item(i) for i in indices]
        batch = self.collator(items)
        if self.target_device_type == "cuda" and torch.cuda.is_available():
            batch = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        return batch

    def __getitem__(self, index: int) -> Dict[str, Any]:
        return self._load_batch(index)

    def _iter_batches(self) -> Iterable[Dict[str, Any]]:
        total = self.total_batches
        if total is not None and self.batches_processed >= total:
            return
        depth = max(1, (self.prefetch_factor or 2) * max(self.num_workers, 1))
        readers = self.num_threads if self.num_threads is not None else 4
        read_pool = ThreadPoolExecutor(max_workers=readers, thread_name_prefix="data-read") if readers > 1 else None
        batch_pool = ThreadPoolExecutor(max_workers=min(depth, 4), thread_name_prefix="data-batch")
        window: Dict[Tuple[int, int], Future] = {}
        try:
            while True:
                k, size = self.batches_processed, self.global_batch_size
                total = self.total_batches
                if total is not None and k >= total:
                    return
                # a changed batch size re-addresses every batch: drop what was prefetched under the old size
                for key in [key for key in window if key[1] != size or key[0] < k]:
                    window.pop(key).cancel()
                last = k + depth if total is None else min(k + depth, total)
                for j in range(k, last):
                    if (j, size) not in window:
                        window[(j, size)] = batch_pool.submit(self._load_batch, j, read_pool)
                yield window.pop((k, size)).result()
        finally:
            for fut in window.values():
                fut.cancel()
            batch_pool.shutdown(wait=True, cancel_futures=True)
            if read_pool is not None:
                read_pool.shutdown(wait=True, cancel_futures=True)

    def get_mock_batch(self) -> Dict[str, Any]:
        rng = torch.Generator(device="cpu").manual_seed(self.seed + self.dp_rank)
        L = self.dataset.max_sequence_length
        n = self.rank_batch_size // L
        out: Dict[str, Any] = {"input_ids": torch.randint(0, self.dataset.vocab_size, (n, L), generator=rng)}
        if isinstance(self.dataset, NumpyFSLDatasetBase) and self.dataset._generate_doc_lengths:
            split = torch.randint(2, L - 2, (n,), generator=rng)
            out["doc_lens"] = torch.stack([split, L - split], dim=1)
            out["max_doc_lens"] = out["doc_lens"].max(dim=-1).values.tolist()
        return out


class NumpyFSLDataLoader(NumpyDataLoaderBase):
    """Fixed sequence length: every global batch is ``global_batch_size // sequence_length`` instances, dealt to ranks round-robin."""

    def __init__(self, dataset: NumpyFSLDatasetBase, *, chunk_size: int = 1, **kwargs):
        assert chunk_size >= 1
        super().__init__(dataset, **kwargs)
        self.chunk_size = chunk_size
        if self.rank_batch_size % dataset.sequence_length != 0:
            raise OLMoConfigurationError(
                f"rank batch size (in tokens) {self.rank_batch_size} must be divisible by sequence length {dataset.sequence_length}"
            )

    @property
    def _instances_per_batch(self) -> int:
        return self.global_batch_size // self.dataset.sequence_length  # type: ignore[attr-defined]

    @property
    def total_size(self) -> int:
        """Instances used per epoch (whole batches only)."""
        per = self._instances_per_batch
        return per * (len(self.dataset) // per)

    @property
    def total_batches(self) -> int:
        return len(self.dataset) // self._instances_per_batch

    @property
    def _global_indices_file(self) -> Path:
        name = _fname("global_indices", seed=self.seed if self.shuffle else None, epoch=self.epoch if self.shuffle else None,
                      dataset_size=len(self.dataset), chunk=self.chunk_size if self.chunk_size > 1 else None, v=1)
        return self.work_dir / f"{name}.npy"

    def _build_global_indices(self) -> np.ndarray:
        n = len(self.dataset)
        assert n < np.iinfo(np.uint32).max
        rng = get_rng(self.seed + self.epoch) if self.shuffle else None
        if self.chunk_size == 1:
            indices = np.arange(n, dtype=np.uint32)
            if rng is not None:
                rng.shuffle(indices)
            return indices
        chunks = np.arange(n // self.chunk_size, dtype=np.uint32)
        if rng is not None:
            rng.shuffle(chunks)
        return (chunks[:, None] * self.chunk_size + np.arange(self.chunk_size, dtype=np.uint32)[None, :]).reshape(-1)

    def _local_instance_indices_for_batch(self, batch_index: int) -> np.ndarray:
        per = self._instances_per_batch
        if not 0 <= batch_index < self.total_batches:
            raise IndexError(batch_index)
        row = self.get_global_indices()[batch_index * per: (batch_index + 1) * per]
        return np.asarray(row[self.dp_rank:: self.dp_world_size])

    def state_dict(self) -> Dict[str, Any]:
        sd = super().state_dict()
        sd.update(dataset_type="fsl", sequence_length=self.dataset.sequence_length,  # type: ignore[attr-defined]
                  max_target_sequence_length=self.dataset.max_target_sequence_length)  # type: ignore[attr-defined]
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        # tokens are the invariant: the batch size may differ from the one the checkpoint was written with
        self.batches_processed = self.tokens_processed // self.global_batch_size
        log.info(f"Data loader will resume from batch {self.batches_processed:,d}/{self.total_batches:,d} based on batch "
                 f"size of {self.global_batch_size:,d} tokens")
        if state_dict["dataset_type"] != "fsl":
            raise RuntimeError("Dataset type mismatch: cannot restore variable-sequence-length state into a fixed-length loader")
        if state_dict["max_target_sequence_length"] != self.dataset.max_target_sequence_length:  # type: ignore[attr-defined]
            raise RuntimeError("Restoring an FSL dataset state with a different 'max_target_sequence_length' is not supported")


class NumpyVSLDataLoader(NumpyDataLoaderBase):
    """Variable sequence length: the epoch order is over *batches*; batch ``b`` takes consecutive instances of its bucket."""

    def __init__(self, dataset: NumpyVSLDataset, **kwargs):
        super().__init__(dataset, **kwargs)
        self._batches_per_bucket: Optional[Tuple[Tuple[int, int], ...]] = None
        self._bucket_indices: Optional[Dict[int, np.ndarray]] = None
        if not self.shuffle:
            log.warning("VSL curriculum will be ignored since shuffle=False")
        if self.rank_batch_size < max(self.buckets):
            raise OLMoConfigurationError(
                f"rank batch size ({self.rank_batch_size:,d}) is too small relative to maximum sequence length ({max(self.buckets):,d})"
            )

    @property
    def buckets(self) -> Tuple[int, ...]:
        return tuple(s for s, _ in self.batches_per_bucket)

    @property
    def batches_per_bucket(self) -> Tuple[Tuple[int, int], ...]:
        if self._batches_per_bucket is None:
            self._batches_per_bucket = tuple(self.dataset.curriculum.batches_per_bucket(self.dataset, self.global_batch_size))  # type: ignore
        return self._batches_per_bucket

    @property
    def total_batches(self) -> int:
        return sum(n for _, n in self.batches_per_bucket)

    def _order_dir(self) -> Path:
        return self.work_dir / f"dataset-{self.dataset.fingerprint}" / self.dataset.curriculum.short_str  # type: ignore

    @property
    def _global_indices_file(self) -> Path:
        name = _fname("global_batch_indices", seed=self.seed if self.shuffle else None,
                      epoch=self.epoch if self.shuffle else None, bz=self.global_batch_size)
        return self._order_dir() / f"{name}.npy"

    def _bucket_indices_file(self, seq_len: int) -> Path:
        name = _fname("instance_indices", bucket=seq_len, seed=self.seed if self.shuffle else None,
                      epoch=self.epoch if self.shuffle else None)
        return self._order_dir() / f"{name}.npy"

    def _get_bucket_indices(self, seq_len: int) -> np.ndarray:
        indices = self.dataset.get_instance_bucket(seq_len)  # type: ignore[attr-defined]
        return get_rng(self.seed + self.epoch + seq_len).permutation(indices) if self.shuffle else np.asarray(indices)

    def build_and_save_global_indices(self, in_memory: bool = False) -> None:
        self._bucket_indices = None
        if in_memory:
            self._bucket_indices = {s: self._get_bucket_indices(s) for s, _ in self.dataset.instances_per_bucket}  # type: ignore
        elif self.fs_local_rank == 0:
            for seq_len, n in self.dataset.instances_per_bucket:  # type: ignore[attr-defined]
                path = self._bucket_indices_file(seq_len)
                if not path.is_file():
                    indices = self._get_bucket_indices(seq_len)
                    assert indices.shape[0] == n
                    write_array_to_disk(indices.astype(np.uint32), path)
            self.dataset.curriculum.log_buckets(self.dataset, self.global_batch_size, self.batches_per_bucket)  # type: ignore
        super().build_and_save_global_indices(in_memory=in_memory)

    def _build_global_indices(self) -> np.ndarray:
        if self.shuffle:
            return self.dataset.curriculum.get_batch_indices(self.batches_per_bucket, self.seed + self.epoch)  # type: ignore
        return np.arange(self.total_batches, dtype=np.uint32)

    def _batch_index_to_bucket_batch_index(self, batch_index: int) -> Tuple[int, int]:
        start = 0
        for seq_len, n in self.batches_per_bucket:
            if start <= batch_index < start + n:
                return seq_len, batch_index - start
            start += n
        raise IndexError(f"Batch index '{batch_index}' out of bounds")

    def _local_instance_indices_for_batch(self, batch_index: int) -> np.ndarray:
        seq_len, k = self._batch_index_to_bucket_batch_index(int(self.get_global_indices()[batch_index]))
        per_batch = self.global_batch_size // seq_len
        per_rank = per_batch // self.dp_world_size
        lo = k * per_batch + self.dp_rank * per_rank
        if self._bucket_indices is not None:
            out = self._bucket_indices[seq_len][lo: lo + per_rank]
        else:
            out = load_array_slice(self._bucket_indices_file(seq_len), lo, lo + per_rank, np.uint32)
        assert out.shape[0] == per_rank, f"Expected {per_rank} instances, got {out.shape[0]}"
        return out

    def state_dict(self) -> Dict[str, Any]:
        sd = super().state_dict()
        ds = self.dataset
        sd.update(dataset_type="vsl", vsl_curriculum=ds.curriculum.short_str,  # type: ignore[attr-defined]
                  max_sequence_length=ds.max_sequence_length, min_sequence_length=ds.min_sequence_length)  # type: ignore
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        log.info(f"Data loader will resume from batch {self.batches_processed}/{self.total_batches}")
        ds = self.dataset
        if state_dict["dataset_type"] != "vsl":
            raise RuntimeError("Dataset type mismatch: cannot restore fixed-sequence-length state into a variable-length loader")
        for key, now in (("vsl_curriculum", ds.curriculum.short_str), ("max_sequence_length", ds.max_sequence_length),  # type: ignore
                         ("min_sequence_length", ds.min_sequence_length)):  # type: ignore[attr-defined]
            if state_dict[key] != now:
                raise RuntimeError(f"Restoring dataset state with a different '{key}' is not supported")


L = TypeVar("L", bound=DataLoaderBase)


@dataclass
class DataLoaderConfig(Config, Registrable, Generic[L]):
    """Base of registrable data loader configs."""

    def build(self, *args, **kwargs) -> L:
        raise NotImplementedError


@DataLoaderConfig.register("numpy")
@dataclass
class NumpyDataLoaderConfig(DataLoaderConfig[NumpyDataLoaderBase]):
    global_batch_size: int
    seed: int
    work_dir: Optional[str] = None
    num_threads: Optional[int] = None
    num_workers: int = 0
    prefetch_factor: Optional[int] = None
    target_device_type: Optional[str] = None
    ignore_fingerprint_mismatch: bool = False

    def build(self, dataset: NumpyDatasetBase, *, collator: Optional[DataCollator] = None, mesh=None,
              dp_process_group: Optional[dist.ProcessGroup] = None) -> NumpyDataLoaderBase:
        """``mesh`` (from ``build_world_mesh``) or ``dp_process_group`` tells which ranks share the data."""
        if self.work_dir is not None:
            if is_url(self.work_dir):
                raise OLMoConfigurationError(f"'work_dir' should be a local path, not a URL ('{self.work_dir}').")
            if not dataset.work_dir_set:
                dataset.work_dir = Path(normalize_path(self.work_dir))
        if dp_process_group is None and mesh is not None:
            dp_process_group = get_dp_process_group(mesh)
        dataset.prepare()
        return NumpyDataLoaderBase.wrap_numpy_dataset(
            dataset, global_batch_size=self.global_batch_size,
            collator=collator or DataCollator(pad_token_id=dataset.pad_token_id, vocab_size=dataset.vocab_size),
            work_dir=self.work_dir or dataset.work_dir, dp_world_size=get_world_size(dp_process_group),
            dp_rank=get_rank(dp_process_group), fs_local_rank=get_fs_local_rank(), seed=self.seed,
            num_threads=self.num_threads, num_workers=self.num_workers, prefetch_factor=self.prefetch_factor,
            target_device_type=self.target_device_type or get_default_device().type,
            ignore_fingerprint_mismatch=self.ignore_fingerprint_mismatch,
        )
