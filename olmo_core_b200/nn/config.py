"""Abstract bases of module/model configs (src/olmo_core/nn/config.py:9-43)."""

from abc import abstractmethod
from dataclasses import dataclass

import torch.nn as nn

from ..config import Config

__all__ = ["ModuleConfig", "ModelConfig"]


@dataclass
class ModuleConfig(Config):
    """A config that knows how to build a sub-module."""

    def build(self, *args, **kwargs) -> nn.Module:
        """Build the module this config describes."""
        raise NotImplementedError


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

    @property
    def num_active_params(self) -> int:
        """Parameters that take part in one token's forward pass (all of them unless the model is sparse)."""
        return self.num_params

    @property
    def num_active_non_embedding_params(self) -> int:
        return self.num_non_embedding_params

    def num_flops_per_token(self, seq_len: int) -> int:
        raise NotImplementedError
