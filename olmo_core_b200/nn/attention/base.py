"""
Abstract sequence mixer (attention, recurrent mixers) and its registrable config
(src/olmo_core/nn/attention/base.py:20-80). Concrete configs register under a name (``attention``, ``gated_delta_net``)
so that a block config can name its mixer in YAML / JSON.
"""

from __future__ import annotations

from abc import abstractmethod
from dataclasses import dataclass
from typing import TYPE_CHECKING, Generic, Optional, TypeVar

import torch
import torch.nn as nn

from ...config import Registrable
from ..buffer_cache import BufferCache
from ..config import ModuleConfig

if TYPE_CHECKING:
    from .ring import RingContextParallelStyle, UlyssesContextParallelStyle

__all__ = ["SequenceMixer", "SequenceMixerConfig", "SeqMixer"]


class SequenceMixer(nn.Module):
    """Base of token-mixing modules (attention, recurrent mixers)."""

    @abstractmethod
    def apply_tp(self, tp_mesh, input_layout=None, output_layout=None, use_local_output: bool = True,
                 float8_enabled: bool = False):
        raise NotImplementedError

    @abstractmethod
    def apply_cp(self, cp_mesh, ring: Optional["RingContextParallelStyle"] = None,
                 uly: Optional["UlyssesContextParallelStyle"] = None):
        raise NotImplementedError

    @abstractmethod
    def num_flops_per_token(self, seq_len: int) -> int:
        raise NotImplementedError

    @abstractmethod
    def init_weights(self, *, init_method, d_model: int, block_idx: int, num_blocks: int, std: float = 0.02,
                     generator: Optional[torch.Generator] = None) -> None:
        raise NotImplementedError


SeqMixer = TypeVar("SeqMixer", bound=SequenceMixer)


@dataclass
class SequenceMixerConfig(ModuleConfig, Registrable, Generic[SeqMixer]):
    def num_params(self, d_model: int) -> int:
        raise NotImplementedError

    def build(self, d_model: int, *, layer_idx: int, n_layers: int, init_device: str = "cpu",
              cache: Optional[BufferCache] = None) -> SeqMixer:
        raise NotImplementedError
