"""
Data loader over composable instance sources (behaviour and state of
src/olmo_core/data/composable/data_loader.py:44-680).

Batches are ADDRESSED, not streamed: batch ``k`` of an epoch is rows ``k`` of the epoch's global instance order reshaped
to ``[batches, instances per batch]``, and rank ``r`` takes columns ``r::dp_world_size``. A bounded window of upcoming
batches is assembled by a thread pool; restoring ``batches_processed`` is all it takes to resume mid-epoch, and a
changed batch size or sequence length re-addresses the same token stream.
"""

from __future__ import annotations

import dataclasses
import functools
import logging
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Iterable, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ...aliases import PathOrStr
from ...config import Config, StrEnum
from ...distributed import utils as dist_utils
from ...distributed.parallel import get_dp_process_group
from ...exceptions import OLMoConfigurationError
from ...utils import get_default_device
from ..collator import DataCollator
from ..data_loader import DataLoaderConfig, TextDataLoaderBase
from ..tokenizer import TokenizerConfig
from ..utils import find_periodic_sequences, get_document_lengths, get_rng, memmap_to_write
from .instance_source import InstanceSource
from .utils import SEED_NOT_SET, as_tensor, build_global_indices, format_fname_from_fields, resolve_seed

log = logging.getLogger(__name__)

__all__ = ["InstanceFilterConfig", "ShuffleStrategy", "ComposableDataLoaderConfig", "ComposableDataLoader"]


@dataclass
class InstanceFilterConfig(Config):
    """Instances with a run of at least ``repetition_max_count`` repeats of an n-gram of the given periods are masked."""

    repetition_max_period: int = 13
    repetition_min_period: int = 1
    repetition_max_count: int = 32


class ShuffleStrategy(StrEnum):
    inter_source = "inter_source"  # one shuffle over all sources
    intra_source = "intra_source"  # shuffle within each source, keep the sources in order (a curriculum)
    interleaved_source = "interleaved_source"  # shuffle within each source, then round-robin over the sources


@DataLoaderConfig.register("composable")
@dataclass
class ComposableDataLoaderConfig(DataLoaderConfig["ComposableDataLoader"]):
    tokenizer: Optional[TokenizerConfig] = None
    global_batch_size: Optional[int] = None
    seed: int = dataclasses.field(default_factory=lambda: resolve_seed(SEED_NOT_SET))
    work_dir: Optional[str] = None
    shuffle: bool = True
    shuffle_strategy: Optional[ShuffleStrategy] = None
    sources_per_epoch: int = -1
    num_threads: Optional[int] = None
    num_workers: int = 0
    prefetch_factor: Optional[int] = None
    target_device_type: Optional[str] = None
    generate_doc_lengths: bool = False
    instance_filter_config: Optional[InstanceFilterConfig] = None
    display_source_visualization: bool = True

    def __post_init__(self, *args):
        del args
        if self.sources_per_epoch == 0 or self.sources_per_epoch < -1:
            raise OLMoConfigurationError("'sources_per_epoch' must be -1 (for all sources) or a positive integer.")
        if not self.shuffle and self.shuffle_strategy is not None:
            raise OLMoConfigurationError("'shuffle_strategy' cannot be set if 'shuffle' is False.")

    def build(self, *sources: InstanceSource, collator: Optional[DataCollator] = None,  # type: ignore[override]
              work_dir: Optional[PathOrStr] = None, mesh=None, dp_process_group: Optional[dist.ProcessGroup] = None,
              tokenizer: Optional[TokenizerConfig] = None, global_batch_size: Optional[int] = None
              ) -> "ComposableDataLoader":
        if not sources:
            raise OLMoConfigurationError("At least one 'source' must be provided.")
        if dp_process_group is None and mesh is not None:
            dp_process_group = get_dp_process_group(mesh)
        work_dir = work_dir or self.work_dir
        tokenizer = tokenizer or self.tokenizer
        global_batch_size = global_batch_size if global_batch_size is not None else self.global_batch_size
        for name, value in (("work_dir", work_dir), ("tokenizer", tokenizer), ("global_batch_size", global_batch_size)):
            if value is None:
                raise OLMoConfigurationError(f"'{name}' must be specified.")
        assert tokenizer is not None and work_dir is not None and global_batch_size is not None
        return ComposableDataLoader(
            *sources,
            collator=collator or DataCollator(pad_token_id=tokenizer.pad_token_id, vocab_size=tokenizer.padded_vocab_size()),
            tokenizer=tokenizer, work_dir=work_dir, global_batch_size=global_batch_size,
            dp_world_size=dist_utils.get_world_size(dp_process_group), dp_rank=dist_utils.get_rank(dp_process_group),
            fs_local_rank=dist_utils.get_fs_local_rank(), seed=self.seed, shuffle=self.shuffle,
            shuffle_strategy=self.shuffle_strategy, sources_per_epoch=self.sources_per_epoch,
            num_threads=self.num_threads, num_workers=self.num_workers, prefetch_factor=self.prefetch_factor,
            target_device_type=self.target_device_type or get_default_device().type,
            generate_doc_lengths=self.generate_doc_lengths, instance_filter_config=self.instance_filter_config,
            display_source_visualization=self.display_source_visualization)


class ComposableDataLoader(TextDataLoaderBase):
    Config = ComposableDataLoaderConfig

    def __init__(self, *sources: InstanceSource, collator: DataCollator, tokenizer: TokenizerConfig, work_dir: PathOrStr,
                 global_batch_size: int, dp_world_size: int = 1, dp_rank: int = 0, fs_local_rank: int = 0, seed: int = 0,
                 shuffle: bool = True, shuffle_strategy: Optional[ShuffleStrategy] = None, sources_per_epoch: int = -1,
                 num_threads: Optional[int] = None, num_workers: int = 0, prefetch_factor: Optional[int] = None,
                 target_device_type: str = "cpu", generate_doc_lengths: bool = False,
                 instance_filter_config: Optional[InstanceFilterConfig] = None,
                 display_source_visualization: bool = True):
        if not sources:
            raise OLMoConfigurationError("At least one source must be provided.")
        shapes = {(s.sequence_length, s.max_sequence_length) for s in sources}
        if len(shapes) != 1:
            raise OLMoConfigurationError("All sources must have the same 'sequence_length' and 'max_sequence_length'.")
        (self.sequence_length, self.max_sequence_length), = shapes
        super().__init__(collator=collator, work_dir=Path(work_dir) / "ComposableDataLoader",
                         global_batch_size=global_batch_size, dp_world_size=dp_world_size, dp_rank=dp_rank,
                         fs_local_rank=fs_local_rank)
        if sources_per_epoch == -1:
            sources_per_epoch = len(sources)
        if sources_per_epoch <= 0 or len(sources) % sources_per_epoch != 0:
            raise OLMoConfigurationError("'sources_per_epoch' must divide the number of sources")
        if global_batch_size % (self.sequence_length * dp_world_size) != 0:
            raise OLMoConfigurationError("'global_batch_size' must be a multiple of sequence_length x dp_world_size")
        self.sources = tuple(sources)
        self.tokenizer = tokenizer
        self.seed = seed
        self.shuffle = shuffle
        self.shuffle_strategy = (shuffle_strategy or ShuffleStrategy.inter_source) if shuffle else None
        self.sources_per_epoch = sources_per_epoch
        self.num_threads, self.num_workers, self.prefetch_factor = num_threads, num_workers, prefetch_factor
        self.target_device_type = target_device_type
        self.generate_doc_lengths = generate_doc_lengths
        self.instance_filter_config = instance_filter_config
        self._global_indices: Optional[np.ndarray] = None
        if display_source_visualization and dist_utils.get_rank() == 0:
            for source in self.sources:
                source.visualize()

    # -- sizes ---------------------------------------------------------------------------------------------
    def sources_for_epoch(self, epoch: int) -> Tuple[InstanceSource, ...]:
        groups = len(self.sources) // self.sources_per_epoch
        first = ((epoch - 1) % groups) * self.sources_per_epoch
        return self.sources[first:first + self.sources_per_epoch]

    @property
    def sources_for_this_epoch(self) -> Tuple[InstanceSource, ...]:
        return self.sources_for_epoch(self._epoch or 1)

    @functools.cached_property
    def source_fingerprints(self) -> Tuple[str, ...]:
        return tuple(s.fingerprint for s in self.sources)

    def instances_in_epoch(self, epoch: int) -> int:
        sources = self.sources_for_epoch(epoch)
        if self.shuffle and self.shuffle_strategy == ShuffleStrategy.interleaved_source:
            return min(len(s) for s in sources) * len(sources)  # every source contributes equally
        return sum(len(s) for s in sources)

    @property
    def total_instances(self) -> int:
        return self.instances_in_epoch(self._epoch or 1)

    @property
    def total_tokens(self) -> int:
        return self.total_instances * self.sequence_length

    def batches_in_epoch(self, epoch: int) -> Optional[int]:
        return self.instances_in_epoch(epoch) // (self.global_batch_size // self.sequence_length)

    @property
    def total_batches(self) -> Optional[int]:
        return self.batches_in_epoch(self._epoch or 1)

    # -- state ---------------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return dict(source_fingerprints=self.source_fingerprints, batches_processed=self.batches_processed,
                    tokens_processed=self.tokens_processed, global_batch_size=self.global_batch_size,
                    sequence_length=self.sequence_length, max_sequence_length=self.max_sequence_length,
                    shuffle=self.shuffle, shuffle_strategy=self.shuffle_strategy,
                    sources_per_epoch=self.sources_per_epoch, seed=self.seed, epoch=self._epoch)

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        if state_dict["sources_per_epoch"] != self.sources_per_epoch:
            raise RuntimeError("Restoring data loader state with a different 'sources_per_epoch' is not supported!")
        saved = tuple(state_dict["source_fingerprints"])
        if saved != self.source_fingerprints:
            # sources may be APPENDED as long as the run has not yet wrapped around the original ones
            appended = len(saved) < len(self.source_fingerprints) and saved == self.source_fingerprints[:len(saved)]
            if not appended:
                raise RuntimeError("Restoring data loader state from different dataset source is not supported "
                                   "(fingerprints don't match)!")
            if state_dict["epoch"] is not None and state_dict["epoch"] > len(saved) // self.sources_per_epoch:
                raise RuntimeError("Restoring data loader state after appending new sources can only be done when the "
                                   "original sources haven't been iterated over yet!")
        for key in ("max_sequence_length", "shuffle_strategy", "shuffle"):
            if state_dict[key] != getattr(self, key):
                raise RuntimeError(f"Restoring data loading state with a different '{key}' is not supported!")
        self.tokens_processed = state_dict["tokens_processed"]
        self.batches_processed = self.tokens_processed // self.global_batch_size
        if state_dict["seed"] != self.seed and self.shuffle:
            log.warning("Restoring data loading state with a different data seed, will use data seed from state dict "
                        "for data order consistency.")
            self.seed = state_dict["seed"]
        self._epoch = state_dict["epoch"] or self._epoch
        self._global_indices = None

    # -- order -----------------------------------------------------------------------------------------------
    def reshuffle(self, epoch: Optional[int] = None, **kwargs) -> None:
        del kwargs
        if epoch is None:
            epoch = 1 if self._epoch is None else self._epoch + 1
        if epoch <= 0:
            raise ValueError(f"'epoch' must be at least 1, got {epoch}")
        self._epoch = epoch
        self.build_and_save_global_indices()

    @property
    def global_indices_file(self) -> Path:
        fingerprint = functools.reduce(lambda a, b: a ^ b, (int(f[:12], 16) for f in
                                                            (s.fingerprint for s in self.sources_for_this_epoch)))
        name = format_fname_from_fields(
            "global_indices", seed=self.seed if self.shuffle else None, epoch=self.epoch if self.shuffle else None,
            shuffle=self.shuffle_strategy if self.shuffle else None, size=self.total_instances,
            seq_len=self.sequence_length, max_seq_len=self.max_sequence_length, src=f"{fingerprint:x}", v=1)
        return self.work_dir / f"{name}.npy"

    def _build_global_indices(self) -> np.ndarray:
        common = dict(sequence_length=self.sequence_length, max_sequence_length=self.max_sequence_length, dtype=np.uint32)
        if not self.shuffle or self.shuffle_strategy == ShuffleStrategy.inter_source:
            return build_global_indices(self.total_instances, seed=(self.seed + self.epoch) if self.shuffle else None,
                                        **common)
        sources = self.sources_for_this_epoch
        offsets = np.concatenate([[0], np.cumsum([len(s) for s in sources])[:-1]])
        if self.shuffle_strategy == ShuffleStrategy.intra_source:
            return np.concatenate([build_global_indices(len(s), seed=self.seed + self.epoch + i, **common) + np.uint32(off)
                                   for i, (s, off) in enumerate(zip(sources, offsets))])
        if self.shuffle_strategy == ShuffleStrategy.interleaved_source:
            per_source = min(len(s) for s in sources)
            out = np.empty(per_source * len(sources), dtype=np.uint32)
            for i, off in enumerate(offsets):
                out[i::len(sources)] = build_global_indices(per_source, seed=self.seed + self.epoch + i, **common) + np.uint32(off)
            return out
        raise NotImplementedError(f"Unknown shuffle strategy: {self.shuffle_strategy}")

    def build_and_save_global_indices(self) -> None:
        self._global_indices = None
        if self.fs_local_rank == 0 and not self.global_indices_file.is_file():
            order = self._build_global_indices()
            self.global_indices_file.parent.mkdir(parents=True, exist_ok=True)
            with memmap_to_write(self.global_indices_file, shape=order.shape, dtype=np.uint32) as mm:
                mm[:] = order
            log.info("Global data order indices saved to '%s'", self.global_indices_file)
        dist_utils.barrier()

    def get_global_indices(self) -> np.ndarray:
        if self._global_indices is None:
            if not self.global_indices_file.is_file():
                raise RuntimeError("Missing global indices file, did you forget to call 'reshuffle()'?")
            self._global_indices = np.memmap(self.global_indices_file, mode="r", dtype=np.uint32)
        return self._global_indices

    def _local_instance_indices_for_batch(self, batch_index: int) -> np.ndarray:
        per_batch = self.global_batch_size // self.sequence_length
        row = self.get_global_indices()[batch_index * per_batch:(batch_index + 1) * per_batch]
        return np.asarray(row[self.dp_rank::self.dp_world_size])

    def get_local_indices(self) -> np.ndarray:
        """This rank's instance indices for the rest of the epoch, in order."""
        total = self.total_batches or 0
        rows = [self._local_instance_indices_for_batch(k) for k in range(self.batches_processed, total)]
        return np.concatenate(rows) if rows else np.empty(0, dtype=np.uint32)

    # -- instances and batches -------------------------------------------------------------------------------------
    def get_instance(self, idx: int) -> Dict[str, Any]:
        if idx < 0:
            idx += self.total_instances
        base = 0
        for source in self.sources_for_this_epoch:
            if idx < base + len(source):
                item = source[idx - base]
                ids = as_tensor(item["input_ids"])
                out: Dict[str, Any] = {"index": idx, "input_ids": ids}
                if source.label is not None:
                    out["metadata"] = {"source": source.label}
                if item.get("label_mask") is not None:
                    out["label_mask"] = as_tensor(item["label_mask"])
                if self.generate_doc_lengths:
                    out["doc_lens"] = get_document_lengths(ids, self.tokenizer.eos_token_id,
                                                           bos_token_id=self.tokenizer.bos_token_id)
                if (f := self.instance_filter_config) is not None:
                    out["instance_mask"] = not any(
                        m.times >= f.repetition_max_count
                        for m in find_periodic_sequences(ids.numpy(), max_period=f.repetition_max_period,
                                                         min_period=f.repetition_min_period))
                return out
            base += len(source)
        raise IndexError(f"Index {idx} out of range for {self.total_instances} instances")

    def _load_batch(self, batch_index: int, pool: Optional[ThreadPoolExecutor] = None) -> Dict[str, Any]:
        indices = [int(i) for i in self._local_instance_indices_for_batch(batch_index)]
        items = list(pool.map(self.get_instance, indices)) if pool is not None else [self.get_instance(i) for i in indices]
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
                for key in [key for key in window if key[1] != size or key[0] < k]:
                    window.pop(key).cancel()  # a changed batch size re-addresses every batch
                for j in range(k, min(k + depth, total if total is not None else k + depth)):
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
        rng = get_rng(self.seed + self.dp_rank)
        n = self.rank_batch_size // self.sequence_length
        return self.collator([self.get_instance(int(i)) for i in rng.integers(0, self.total_instances, n)])
