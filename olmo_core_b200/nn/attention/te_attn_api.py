"""Transformer-Engine attention is not used by this framework (name of src/olmo_core/nn/attention/te_attn_api.py:7)."""

__all__ = ["has_te_attn"]


def has_te_attn() -> bool:
    return False
