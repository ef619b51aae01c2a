"""Next-token selection: greedy, temperature, top-k and nucleus filtering (src/olmo_core/generate/sampling.py)."""

import torch

__all__ = ["greedy_selection", "top_k_filtering", "top_p_filtering", "select_next_token"]


def greedy_selection(logits: torch.Tensor) -> torch.Tensor:
    return logits.argmax(dim=-1)


def top_k_filtering(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """Keep the ``top_k`` largest logits of every row, set the others to ``-inf``."""
    if top_k <= 0:
        return logits
    kth = torch.topk(logits, k=min(top_k, logits.size(-1)), dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_filtering(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    """Keep the smallest set of tokens whose probability mass reaches ``top_p`` (always at least one)."""
    if top_p <= 0.0 or top_p >= 1.0:
        return logits
    sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
    mass_before = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1) - torch.softmax(sorted_logits, dim=-1)
    drop_sorted = mass_before > top_p  # a token goes once the tokens ranked above it already exceed the threshold
    drop = torch.zeros_like(drop_sorted).scatter(-1, order, drop_sorted)
    return logits.masked_fill(drop, float("-inf"))


def select_next_token(logits: torch.Tensor, do_sample: bool = True, temperature: float = 0.0, top_k: int = -1,
                      top_p: float = 1.0, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``logits [..., vocab] -> token ids [...]``; ``temperature == 0`` or ``do_sample=False`` means greedy."""
    if not do_sample or temperature == 0:
        return greedy_selection(logits)
    if torch.isnan(logits).any():
        bad = [i for i in range(logits.shape[0]) if torch.isnan(logits[i]).any()]
        raise AssertionError(f"NaN values detected in logits of shape {tuple(logits.shape)} in batch elements {bad}")
    scaled = logits / temperature
    if top_k != -1:
        scaled = top_k_filtering(scaled, top_k)
    if top_p != 1.0:
        scaled = top_p_filtering(scaled, top_p)
    probs = torch.softmax(scaled, dim=-1, dtype=dtype)
    flat = torch.multinomial(probs.reshape(-1, probs.shape[-1]), num_samples=1).squeeze(-1)
    return flat.reshape(probs.shape[:-1])
