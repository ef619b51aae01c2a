"""Base class of train-module configs (counterpart of src/olmo_core/train/train_module/config.py).

A train-module config is the serialisable description of how a model is trained (optimizer, micro-batch size,
parallelism, precision); ``build`` turns it into the live ``TrainModule`` around an already constructed model.
"""

from dataclasses import dataclass

from ...config import Config

__all__ = ["TrainModuleConfig"]


@dataclass
class TrainModuleConfig(Config):
    def build(self, *args, **kwargs):
        """Return the train module; concrete configs take the model (and optionally a device) as arguments."""
        raise NotImplementedError(f"{type(self).__name__} does not define build()")
