"""Interface of generation modules (src/olmo_core/generate/generation_module/generation_module.py)."""

from abc import ABCMeta, abstractmethod
from typing import Any, Dict, Optional, Tuple

import torch

__all__ = ["GenerationModule"]


class GenerationModule(metaclass=ABCMeta):
    @property
    def dp_process_group(self):
        """The data-parallel process group generation runs on (``None``: every rank generates on its own replica)."""
        return None

    @abstractmethod
    def generate_batch(self, input_ids: torch.Tensor, *, attention_mask: Optional[torch.Tensor] = None,
                       **kwargs) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        """``(token ids, logits or None, log-probabilities or None)``."""
        raise NotImplementedError

    @abstractmethod
    def state_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def state_dict_to_load(self, metadata) -> Dict[str, Any]:
        """The state dict to fill when loading a checkpoint described by ``metadata``; by default :meth:`state_dict`."""
        del metadata
        return self.state_dict()

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        raise NotImplementedError
