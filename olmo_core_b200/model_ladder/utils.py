"""Human-readable counts for ladder reports (src/olmo_core/model_ladder/utils.py:1-11)."""

from ..utils import format_int

__all__ = ["format_count", "format_tokens"]


def format_count(count: int) -> str:
    return format_int(count)


def format_tokens(tokens: int) -> str:
    return f"{format_count(tokens)} tokens"
