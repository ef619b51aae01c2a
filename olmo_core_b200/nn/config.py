"""Abstract bases of module/model configs (src/olmo_core/nn/config.py:9-43)."""

from abc import abstractmethod
from dataclasses import dataclass

import torch.nn as nn

from ..config import Config

__all__ = ["ModuleConfig", "ModelConfig"]


@dataclass
class ModuleConfig(Config):
    """A config that knows how to build a sub-module."""


@dataclass
class ModelConfig(Config):
    """A config that builds a whole model and can count its parameters."""

    @abstractmethod
    def build(self, *, init_device: str = "cpu") -> nn.Module:
        raise NotImplementedError

    @property
    @abstractmethod
    def num_params(self) -> int:
        raise NotImplementedError

    @property
    @abstractmethod
    def num_non_embedding_params(self) -> int:
        raise NotImplementedError

    def num_flops_per_token(self, seq_len: int) -> int:
        raise NotImplementedError
