"""Interface of generation modules (src/olmo_core/generate/generation_module/generation_module.py)."""

from abc import ABCMeta, abstractmethod
from typing import Any, Dict, Optional, Tuple

import torch

__all__ = ["GenerationModule"]


class GenerationModule(metaclass=ABCMeta):
    @abstractmethod
    def generate_batch(self, input_ids: torch.Tensor, *, attention_mask: Optional[torch.Tensor] = None,
                       **kwargs) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        """``(token ids, logits or None, log-probabilities or None)``."""
        raise NotImplementedError

    @abstractmethod
    def state_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    @abstractmethod
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        raise NotImplementedError
