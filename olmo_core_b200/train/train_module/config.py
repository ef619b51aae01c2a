from abc import abstractmethod
from dataclasses import dataclass

from ...config import Config

__all__ = ["TrainModuleConfig"]


@dataclass
class TrainModuleConfig(Config):
    """Base of train-module configs (src/olmo_core/train/train_module/config.py)."""

    @abstractmethod
    def build(self, *args, **kwargs):
        raise NotImplementedError
