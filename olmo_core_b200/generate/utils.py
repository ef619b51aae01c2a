"""Helpers for generation (src/olmo_core/generate/utils.py)."""

import torch

__all__ = ["selective_log_softmax"]


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., index]`` without materialising the full log-softmax: ``logit - logsumexp``."""
    logits = logits.float()
    picked = torch.gather(logits, dim=-1, index=index.unsqueeze(-1) if index.dim() < logits.dim() else index).squeeze(-1)
    return picked - torch.logsumexp(logits, dim=-1)
