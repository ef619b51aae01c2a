"""Hugging Face config for a transformer built with this framework (role of src/olmo_core/nn/hf/config.py)."""

from __future__ import annotations

from typing import Any, Dict, Optional

__all__ = ["get_hf_config"]


def _rope_scaling(rope) -> Optional[Dict[str, Any]]:
    scaling = getattr(rope, "scaling", None)
    if scaling is None:
        return None
    if hasattr(scaling, "to_hf_dict"):
        return scaling.to_hf_dict()
    out = {k: v for k, v in vars(scaling).items() if not k.startswith("_") and v is not None}
    out.setdefault("rope_type", type(scaling).__name__.replace("RoPEScalingConfig", "").lower() or "default")
    return out


def get_hf_config(model):
    """``Olmo2Config`` (``Olmo3Config`` with sliding windows) for reordered-norm blocks, ``LlamaConfig`` for pre-norm blocks."""
    from transformers import LlamaConfig, Olmo2Config

    from ..transformer.block import ReorderedNormTransformerBlock
    from ..transformer.model import MoETransformer, NormalizedTransformer

    if isinstance(model, NormalizedTransformer):
        raise NotImplementedError(f"Building HF config not implemented for {type(model).__name__}")
    if isinstance(model, MoETransformer):
        raise NotImplementedError("Mixture-of-experts export uses the expert templates of nn.hf.convert; build the HF "
                                  "config for the target architecture explicitly")
    blocks = list(model.blocks.values())
    first = blocks[0]
    attn = first.attention
    common = dict(
        vocab_size=model.vocab_size, hidden_size=model.d_model, intermediate_size=first.feed_forward.hidden_size,
        num_hidden_layers=model.n_layers, num_attention_heads=attn.n_heads, num_key_value_heads=attn.n_kv_heads,
        hidden_act="silu", max_position_embeddings=-1, attention_bias=attn.w_out.bias is not None,
        rope_theta=attn.rope.theta if attn.rope is not None else None,
        rope_scaling=_rope_scaling(attn.rope) if attn.rope is not None else None,
        pad_token_id=None, bos_token_id=None, eos_token_id=None, rms_norm_eps=first.feed_forward_norm.eps,
        tie_word_embeddings=getattr(model, "tie_word_embeddings", False),
    )
    if not isinstance(first, ReorderedNormTransformerBlock):
        return LlamaConfig(**common)
    windows = {b.attention.window_size for b in blocks if getattr(b.attention, "window_size", None)}
    if windows:
        try:
            from transformers import Olmo3Config
        except ImportError as e:
            raise RuntimeError("The installed transformers version does not support Olmo3") from e
        if len(windows) > 1:
            raise ValueError(f"All sliding-window layers must share one window size, found {windows}")
        layer_types = ["sliding_attention" if getattr(b.attention, "window_size", None) else "full_attention" for b in blocks]
        return Olmo3Config(**common, sliding_window=windows.pop(), layer_types=layer_types)
    return Olmo2Config(**common)


def __getattr__(name: str):
    # defined in ``hybrid.py``; reachable under this module's name as well
    if name in ('is_olmo_hybrid_model', 'get_hybrid_layer_types', 'get_hybrid_hf_config'):
        from . import hybrid

        return getattr(hybrid, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
