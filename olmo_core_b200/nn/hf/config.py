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


def _moe_hf_config(model):
    """
    Mixture-of-experts models: ``FlexOlmoConfig`` for reordered-norm blocks (norms on the sub-layer outputs, as in OLMo-2),
    ``OlmoeConfig`` for pre-norm blocks. Both Hugging Face architectures route with a softmax over all experts followed
    by top-k, one SwiGLU MLP per expert and no shared expert; anything else has no counterpart there.
    """
    from ..transformer.block import MoEReorderedNormTransformerBlock

    blocks = list(model.blocks.values())
    first = blocks[0]
    if any(not hasattr(b, "feed_forward_moe") or hasattr(b, "feed_forward") for b in blocks):
        raise NotImplementedError("only models whose every block is a pure mixture-of-experts block can be exported")
    moe, attn = first.feed_forward_moe, first.attention
    router = moe.router
    if getattr(moe, "shared_mlp", None) is not None:
        raise NotImplementedError("shared experts have no counterpart in the Hugging Face OLMoE / FlexOlmo architectures")
    if str(getattr(router, "gating_function", "softmax")).split(".")[-1] != "softmax":
        raise NotImplementedError("only softmax routers can be exported")
    common = dict(
        vocab_size=model.vocab_size, hidden_size=model.d_model, intermediate_size=moe.experts.mlp.hidden_size,
        num_hidden_layers=model.n_layers, num_attention_heads=attn.n_heads, num_key_value_heads=attn.n_kv_heads,
        hidden_act="silu", max_position_embeddings=-1, attention_bias=attn.w_out.bias is not None,
        pad_token_id=None, bos_token_id=None, eos_token_id=None, rms_norm_eps=first.feed_forward_norm.eps,
        tie_word_embeddings=getattr(model, "tie_word_embeddings", False), num_experts=moe.num_experts,
        num_experts_per_tok=router.top_k, norm_topk_prob=bool(getattr(router, "normalize_expert_weights", None)),
    )
    rope = attn.rope
    if isinstance(first, MoEReorderedNormTransformerBlock):
        from transformers import FlexOlmoConfig

        params = {"rope_type": "default", "rope_theta": rope.theta} if rope is not None else None
        scaling = _rope_scaling(rope) if rope is not None else None
        if scaling:
            params = {**scaling, "rope_theta": rope.theta}
        return FlexOlmoConfig(**common, rope_parameters=params)
    from transformers import OlmoeConfig

    return OlmoeConfig(**common, rope_theta=rope.theta if rope is not None else None,
                       rope_scaling=_rope_scaling(rope) if rope is not None else None)


def _gemma3_hf_config(model, blocks, common):
    """Peri-norm blocks (norms on both sides of each sub-layer), GeGLU, local / global attention layers: Gemma-3 text."""
    from transformers import Gemma3TextConfig

    first = blocks[0].attention
    layer_types = ["sliding_attention" if getattr(b.attention, "window_size", None) else "full_attention" for b in blocks]
    windows = {b.attention.window_size for b in blocks if getattr(b.attention, "window_size", None)}
    if len(windows) > 1:
        raise ValueError(f"All sliding-window layers must share one window size, found {windows}")
    thetas = {kind: next((b.attention.rope.theta for b, t in zip(blocks, layer_types) if t == kind and b.attention.rope is not None), None)
              for kind in ("sliding_attention", "full_attention")}
    params = {k: v for k, v in common.items() if k not in ("rope_theta", "rope_scaling", "hidden_act", "attention_bias")}
    return Gemma3TextConfig(
        **params, head_dim=first.head_dim, hidden_activation="gelu_pytorch_tanh", query_pre_attn_scalar=first.head_dim,
        sliding_window=windows.pop() if windows else None, layer_types=layer_types,
        rope_parameters={kind: {"rope_type": "default", "rope_theta": float(theta)} for kind, theta in thetas.items() if theta},
        final_logit_softcapping=None, attn_logit_softcapping=None,
    )


def get_hf_config(model):
    """
    ``Olmo2Config`` (``Olmo3Config`` with sliding windows) for reordered-norm blocks, ``Gemma3TextConfig`` for peri-norm
    blocks, ``Qwen3Config`` for pre-norm blocks with per-head query / key norms, ``LlamaConfig`` for other pre-norm blocks.
    """
    from transformers import LlamaConfig, Olmo2Config

    from ..transformer.block import ReorderedNormTransformerBlock
    from ..transformer.model import MoETransformer, NormalizedTransformer

    if isinstance(model, NormalizedTransformer):
        raise NotImplementedError(f"Building HF config not implemented for {type(model).__name__}")
    if isinstance(model, MoETransformer):
        return _moe_hf_config(model)
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
    if hasattr(first, "post_attention_norm") and hasattr(first, "post_feed_forward_norm"):
        return _gemma3_hf_config(model, blocks, common)
    if not isinstance(first, ReorderedNormTransformerBlock):
        if getattr(attn, "use_head_qk_norm", False) and attn.q_norm is not None:
            from transformers import Qwen3Config

            # pre-norm blocks with a per-head RMSNorm on queries and keys: the Qwen-3 architecture
            params = dict(common)
            theta, scaling = params.pop("rope_theta"), params.pop("rope_scaling")
            return Qwen3Config(**params, head_dim=attn.head_dim, rope_parameters={**(scaling or {"rope_type": "default"}),
                                                                                    "rope_theta": theta})
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
