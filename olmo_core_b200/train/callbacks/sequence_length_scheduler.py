"""
Sequence-length warm-up (behaviour of src/olmo_core/train/callbacks/sequence_length_scheduler.py:18-180).

During the first ``warmup_steps`` steps each batch is reshaped to a shorter sequence length that grows linearly
from ``min_sequence_length`` to the data loader's length: either *melted* -- every sequence split into
``2**k`` shorter ones, keeping all tokens, with the micro-batch size scaled so that tokens per micro-batch stay
constant -- or *truncated* to a multiple of ``keep_multiple_of``.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

from ...data.utils import melt_batch, truncate_batch
from ...exceptions import OLMoConfigurationError
from ...utils import gc_cuda
from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["SequenceLengthSchedulerCallback", "split_sequence_length", "truncated_sequence_length"]


def _linear(min_len: int, max_len: int, step: int, warmup_steps: int) -> float:
    return min_len + (max_len - min_len) * min(step, warmup_steps) / warmup_steps


def split_sequence_length(min_len: int, max_len: int, step: int, warmup_steps: int) -> int:
    """Largest ``min_len * 2**n`` not above the linear ramp."""
    n = math.floor(math.log2(_linear(min_len, max_len, step, warmup_steps) // min_len))
    return min_len * 2**n


def truncated_sequence_length(min_len: int, max_len: int, step: int, warmup_steps: int, keep_multiple_of: int) -> int:
    return int(keep_multiple_of * (_linear(min_len, max_len, step, warmup_steps) // keep_multiple_of))


@dataclass
class SequenceLengthSchedulerCallback(Callback):
    min_sequence_length: int = 128
    warmup_steps: int = 2000
    truncate: bool = False
    keep_multiple_of: int = 128
    enabled: bool = True

    _og_rank_microbatch_size: Optional[int] = None
    _last_seq_len: Optional[int] = None

    def _max_len(self) -> int:
        dataset = getattr(self.trainer.data_loader, "dataset", None)
        seq_len = getattr(dataset, "sequence_length", None) or getattr(self.trainer.train_module, "max_sequence_length", None)
        if seq_len is None:
            raise OLMoConfigurationError("The sequence length scheduler needs a fixed-sequence-length data loader")
        return seq_len

    def pre_train(self) -> None:
        if not self.enabled:
            return
        if not hasattr(self.trainer.train_module, "rank_microbatch_size"):
            raise OLMoConfigurationError("The sequence length scheduler needs a train module with 'rank_microbatch_size'")
        max_len = self._max_len()
        if max_len <= self.min_sequence_length:
            raise OLMoConfigurationError("train sequence length must be greater than 'min_sequence_length'")
        if not self.truncate:
            ratio = max_len / self.min_sequence_length
            if max_len % self.min_sequence_length != 0 or math.log2(ratio) % 1 != 0:
                raise OLMoConfigurationError(
                    "train sequence length must be a multiple of 'min_sequence_length' by a power of 2 when 'truncate=False'"
                )
        self._og_rank_microbatch_size = self.trainer.train_module.rank_microbatch_size

    def pre_step(self, batch: Dict[str, Any]) -> None:
        if not self.enabled or self.step > self.warmup_steps:
            return
        max_len = self._max_len()
        if self.truncate:
            new_len = truncated_sequence_length(self.min_sequence_length, max_len, self.step, self.warmup_steps,
                                                self.keep_multiple_of)
            batch.update(truncate_batch(batch, new_len))
        else:
            new_len = split_sequence_length(self.min_sequence_length, max_len, self.step, self.warmup_steps)
            batch.update(melt_batch(batch, new_len))
            assert self._og_rank_microbatch_size is not None
            self.trainer.train_module.rank_microbatch_size = self._og_rank_microbatch_size * (max_len // new_len)
        if new_len != self._last_seq_len:
            log.info(f"Changing sequence length to {new_len} per warm-up schedule")
            self._last_seq_len = new_len
            gc_cuda()  # activation shapes changed: release cached blocks of the old sizes

    def post_train_batch(self) -> None:
        if not self.enabled or self.step > self.warmup_steps + 1 or self._og_rank_microbatch_size is None:
            return
        self.trainer.train_module.rank_microbatch_size = self._og_rank_microbatch_size
