"""Generation settings (src/olmo_core/generate/generation_module/config.py)."""

from dataclasses import dataclass
from typing import List, Optional

from ...config import Config

__all__ = ["GenerationConfig"]


@dataclass
class GenerationConfig(Config):
    pad_token_id: int
    eos_token_id: int
    max_length: Optional[int] = None
    """Upper bound on prompt + generated tokens."""
    max_new_tokens: Optional[int] = None
    """Upper bound on generated tokens; takes precedence over ``max_length``."""
    do_sample: bool = True
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    use_cache: bool = True
    stop_token_ids: Optional[List[int]] = None

    def __post_init__(self):
        self.validate()

    def validate(self) -> None:
        if self.pad_token_id < 0:
            raise ValueError(f"pad_token_id must be non-negative, got {self.pad_token_id}")
        if self.eos_token_id < 0:
            raise ValueError(f"eos_token_id must be non-negative, got {self.eos_token_id}")
        if self.pad_token_id == self.eos_token_id:
            raise ValueError(f"pad_token_id and eos_token_id must be different, got {self.pad_token_id} and {self.eos_token_id}")
        if self.max_length is not None and self.max_length <= 0:
            raise ValueError(f"max_length must be positive, got {self.max_length}")
        if self.max_new_tokens is not None and self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be positive, got {self.max_new_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}")
        if self.top_k <= 0 and self.top_k != -1:
            raise ValueError(f"top_k must be positive or -1, got {self.top_k}")
        if self.top_p <= 0.0 or self.top_p > 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
