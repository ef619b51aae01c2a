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
        """Reject settings that no sampler can honour. All problems are reported at once."""
        problems = []

        def require(ok: bool, what: str) -> None:
            if not ok:
                problems.append(what)

        for name in ("pad_token_id", "eos_token_id"):
            require(getattr(self, name) >= 0, f"{name}={getattr(self, name)} is not a token id (negative)")
        require(self.pad_token_id != self.eos_token_id,
                f"pad_token_id and eos_token_id are both {self.pad_token_id}; padding could not be told from the end of text")
        for name in ("max_length", "max_new_tokens"):
            value = getattr(self, name)
            require(value is None or value > 0, f"{name}={value} leaves no room for tokens")
        require(self.temperature >= 0, f"temperature={self.temperature} is below zero")
        require(self.top_k == -1 or self.top_k > 0, f"top_k={self.top_k}: use -1 to switch it off or a count of at least 1")
        require(0.0 < self.top_p <= 1.0, f"top_p={self.top_p} lies outside (0, 1]")
        if problems:
            raise ValueError("invalid generation settings: " + "; ".join(problems))
