"""
How to set up a transformer of a given nominal size on a given device type
(behaviour of src/olmo_core/model_ladder/transformer_model_configurator.py:25-277).

Micro-batch sizes are per device, in tokens, for 80 GB H100s; a B200 (180 GB) takes twice as much. Models below 13B
need at least 8 devices, larger ones 32.
"""

from __future__ import annotations

import dataclasses
import re
from dataclasses import dataclass
from typing import Any, Dict, Optional

from ..config import DType, StrEnum
from ..data import TokenizerConfig
from ..distributed.parallel import DataParallelType
from ..exceptions import OLMoConfigurationError
from ..nn.attention import AttentionBackendName
from ..nn.transformer import TransformerConfig
from ..optim import OptimConfig, Scheduler
from ..train.train_module import (
    TransformerDataParallelConfig,
    TransformerDataParallelWrappingStrategy,
    TransformerTrainModule,
    TransformerTrainModuleConfig,
)
from ..utils import warn_once
from .base import DeviceMeshSpec, ModelConfigurator
from .utils import format_count

__all__ = ["TransformerSize", "TransformerModelConfigurator", "Olmo3ModelConfigurator"]

_UNITS = {"K": 1e3, "M": 1e6, "B": 1e9, "T": 1e12}
# (largest parameter count the row applies to, sequences of 4096 tokens per device on an H100)
_MICROBATCH_TABLE = [(100e6, 4), (190e6, 16), (370e6, 12), (760e6, 10), (1e9, 8), (3e9, 4), (7e9, 2), (float("inf"), 2)]
_SUPPORTED_SEQ_LENS = (2048, 4096, 8192)


class TransformerSize(StrEnum):
    size_60M = "60M"
    size_100M = "100M"
    size_190M = "190M"
    size_370M = "370M"
    size_600M = "600M"
    size_760M = "760M"
    size_1B = "1B"
    size_3B = "3B"
    size_7B = "7B"
    size_13B = "13B"

    @property
    def approx_num_params(self) -> int:
        m = re.fullmatch(r"([\d.]+)([KMBT])", self.value.replace(" ", "").upper())
        if m is None:
            raise ValueError(f"Invalid size descriptor '{self}'")
        return int(float(m.group(1)) * _UNITS[m.group(2)])

    def _cmp(self, other, op):
        if isinstance(other, TransformerSize):
            return op(self.approx_num_params, other.approx_num_params)
        return op(str(self), other)

    def __lt__(self, other) -> bool:  # ordered by size, not alphabetically
        return self._cmp(other, lambda a, b: a < b)

    def __le__(self, other) -> bool:
        return self._cmp(other, lambda a, b: a <= b)

    def __gt__(self, other) -> bool:
        return self._cmp(other, lambda a, b: a > b)

    def __ge__(self, other) -> bool:
        return self._cmp(other, lambda a, b: a >= b)


def _check(device_type: str, sequence_length: int) -> str:
    device_type = device_type.lower()
    if not ("h100" in device_type or "b200" in device_type):
        raise OLMoConfigurationError(f"no settings for device type '{device_type}' (H100 and B200 are covered)")
    if sequence_length not in _SUPPORTED_SEQ_LENS:
        raise OLMoConfigurationError(f"sequence length must be one of {_SUPPORTED_SEQ_LENS}")
    return device_type


@dataclass(kw_only=True, eq=True)
class TransformerModelConfigurator(ModelConfigurator[TransformerConfig]):
    rank_microbatch_size: Optional[int] = None  # fixed value in tokens; otherwise derived from size and device

    def configure_rank_microbatch_size(self, *, size_spec: str, sequence_length: int, device_type: str) -> int:
        if self.rank_microbatch_size is not None:
            if self.rank_microbatch_size <= 0 or self.rank_microbatch_size % sequence_length != 0:
                raise OLMoConfigurationError("rank_microbatch_size must be a positive multiple of the sequence length")
            return self.rank_microbatch_size
        device_type = _check(device_type, sequence_length)
        n = TransformerSize(size_spec).approx_num_params
        sequences = next(s for limit, s in _MICROBATCH_TABLE if n <= limit)
        tokens = sequences * 4096
        return tokens * 2 if "b200" in device_type else tokens

    def configure_minimal_device_mesh_spec(self, *, size_spec: str, sequence_length: int, device_type: str) -> DeviceMeshSpec:
        _check(device_type, sequence_length)
        big = TransformerSize(size_spec).approx_num_params >= 13e9
        return DeviceMeshSpec(world_size=32 if big else 8, dp_world_size=None)

    def build_train_module(self, *, size_spec: str, sequence_length: int, rank_microbatch_size: int,
                           model_config: TransformerConfig, optim_config: OptimConfig, scheduler: Scheduler,
                           device_type: str) -> TransformerTrainModule:
        _check(device_type, sequence_length)
        TransformerSize(size_spec)
        config = TransformerTrainModuleConfig(
            rank_microbatch_size=rank_microbatch_size, max_sequence_length=sequence_length, optim=optim_config,
            compile_model=True, z_loss_multiplier=1e-5, max_grad_norm=1.0, scheduler=scheduler,
            dp_config=TransformerDataParallelConfig(name=DataParallelType.fsdp, param_dtype=DType.bfloat16,
                                                    reduce_dtype=DType.float32,
                                                    wrapping_strategy=TransformerDataParallelWrappingStrategy.full))
        train_module = config.build(model_config.build(init_device="meta"))
        assert isinstance(train_module, TransformerTrainModule)
        return train_module


@dataclass(kw_only=True, eq=True)
class Olmo3ModelConfigurator(TransformerModelConfigurator):
    model_construction_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)

    def configure_model(self, *, size_spec: str, sequence_length: int, tokenizer: TokenizerConfig,
                        device_type: str) -> TransformerConfig:
        device_type = _check(device_type, sequence_length)
        size = TransformerSize(size_spec)
        backend = AttentionBackendName.torch
        wanted = AttentionBackendName.flash_3 if "h100" in device_type else AttentionBackendName.flash_4
        try:
            wanted.assert_supported()
            backend = wanted
        except RuntimeError:
            pass
        factory = getattr(TransformerConfig, f"olmo3_{size.value}", None)
        if factory is None:
            raise OLMoConfigurationError(f"Unsupported model size '{size}'")
        model = factory(tokenizer.padded_vocab_size(), attn_backend=backend, **self.model_construction_kwargs)
        target = size.approx_num_params
        off = abs(model.num_non_embedding_params - target) / target
        if off > 0.05:
            warn_once(f"Configured model has {format_count(model.num_non_embedding_params)} (non-embedding) parameters, "
                      f"which differs from target of {size} by ~{100 * off:.1f}%.", UserWarning)
        return model
