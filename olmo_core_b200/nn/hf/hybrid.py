"""
Hugging Face interchange for hybrid models that mix Gated DeltaNet layers with full-attention layers
(the ``olmo_hybrid`` export of src/olmo_core/nn/hf/config.py:255-411, src/olmo_core/nn/hf/convert.py:800-895 and
src/olmo_core/nn/hf/checkpoint.py:205-267, and the Qwen3.5 import of src/olmo_core/nn/hf/convert.py:440-665).

Both directions are table-driven here: a layer's parameter names are its mixer's table (``linear_attn.*`` for a Gated
DeltaNet layer, ``self_attn.*`` for attention) plus one MLP table, because the two layer kinds share the
``blocks.{i}.attention.*`` prefix on this side but not on the Hugging Face side, which rules out one name template per
model. The export writes ``config.json`` and ``model.safetensors`` directly and needs no particular ``transformers``
version.
"""

from __future__ import annotations

import json
import logging
import re
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch

from ...aliases import PathOrStr
from ...config import DType

log = logging.getLogger(__name__)

__all__ = [
    "is_olmo_hybrid_model",
    "get_hybrid_layer_types",
    "get_hybrid_hf_config",
    "convert_hybrid_state_to_hf",
    "save_hf_hybrid_model",
    "convert_qwen3_5_state_from_hf",
]

LINEAR, FULL = "linear_attention", "full_attention"

_MLP = {"feed_forward.w1.weight": "mlp.gate_proj.weight", "feed_forward.w2.weight": "mlp.down_proj.weight",
        "feed_forward.w3.weight": "mlp.up_proj.weight"}
# Gated DeltaNet layers are pre-norm on the Hugging Face side, attention layers post-norm: the two norms of a block land
# on different names.
_LAYER_TABLES: Dict[str, Dict[str, str]] = {
    LINEAR: {
        **{f"attention.{ours}": f"linear_attn.{theirs}" for ours, theirs in (
            ("w_q.weight", "q_proj.weight"), ("w_k.weight", "k_proj.weight"), ("w_v.weight", "v_proj.weight"),
            ("w_a.weight", "a_proj.weight"), ("w_b.weight", "b_proj.weight"), ("w_g.weight", "g_proj.weight"),
            ("w_out.weight", "out_proj.weight"), ("q_conv1d.weight", "q_conv1d.weight"),
            ("k_conv1d.weight", "k_conv1d.weight"), ("v_conv1d.weight", "v_conv1d.weight"),
            ("o_norm.weight", "norm.weight"), ("A_log", "A_log"), ("dt_bias", "dt_bias"))},
        "attention_norm.weight": "input_layernorm.weight",
        "feed_forward_norm.weight": "post_attention_layernorm.weight",
        **_MLP,
    },
    FULL: {
        **{f"attention.{ours}": f"self_attn.{theirs}" for ours, theirs in (
            ("w_q.weight", "q_proj.weight"), ("w_k.weight", "k_proj.weight"), ("w_v.weight", "v_proj.weight"),
            ("w_out.weight", "o_proj.weight"), ("q_norm.weight", "q_norm.weight"), ("k_norm.weight", "k_norm.weight"))},
        "attention_norm.weight": "post_attention_layernorm.weight",
        "feed_forward_norm.weight": "post_feedforward_layernorm.weight",
        **_MLP,
    },
}
_TOP_LEVEL = {"embeddings.weight": "model.embed_tokens.weight", "lm_head.norm.weight": "model.norm.weight",
              "lm_head.w_out.weight": "lm_head.weight"}
_BLOCK_KEY = re.compile(r"^blocks\.(\d+)\.(.+)$")


def _mixer_kind(block) -> Optional[str]:
    from ..attention import Attention
    from ..attention.recurrent import GatedDeltaNet

    if isinstance(block.attention, GatedDeltaNet):
        return LINEAR
    if isinstance(block.attention, Attention):
        return FULL
    return None


def is_olmo_hybrid_model(model) -> bool:
    """True when the model has at least one Gated DeltaNet layer and at least one attention layer."""
    kinds = {_mixer_kind(b) for b in model.blocks.values()}
    return LINEAR in kinds and FULL in kinds


def get_hybrid_layer_types(model) -> List[str]:
    """``"linear_attention"`` / ``"full_attention"`` per layer, the ``layer_types`` field of the ``olmo_hybrid`` config."""
    out = []
    for idx, block in model.blocks.items():
        kind = _mixer_kind(block)
        if kind is None:
            raise ValueError(f"Unknown sequence mixer type at layer {idx}: {type(block.attention)}")
        out.append(kind)
    return out


def _rope_parameters(model, layer_types: List[str]) -> Optional[Dict[str, Any]]:
    """RoPE settings of the attention layers (Gated DeltaNet layers have none); scaled layers must agree."""
    attn_blocks = [b for b, t in zip(model.blocks.values(), layer_types) if t == FULL]
    rope = attn_blocks[0].attention.rope
    if rope is None:
        return None
    scalings = [b.attention.rope.scaling.to_hf_config() for b in attn_blocks
                if b.attention.rope is not None and b.attention.rope.scaling is not None]
    if any(s != scalings[0] for s in scalings[1:]):
        raise NotImplementedError(f"Inconsistent RoPE scaling configs across attention layers: {scalings}")
    params: Dict[str, Any] = {"rope_theta": float(rope.theta)}
    if scalings:
        params.update(scalings[0])
    else:
        params["rope_type"] = "default"
    return params


def get_hybrid_hf_config(model, layer_types: List[str], max_seq_len: int = 65536) -> Dict[str, Any]:
    """The ``config.json`` of a Hugging Face ``olmo_hybrid`` model, as a plain dict."""
    from ..transformer.block import ReorderedNormTransformerBlock

    first = {kind: next((b for b, t in zip(model.blocks.values(), layer_types) if t == kind), None) for kind in (FULL, LINEAR)}
    if first[FULL] is None:
        raise ValueError("Hybrid model must have at least one attention layer")
    if first[LINEAR] is None:
        raise ValueError("Hybrid model must have at least one GDN layer")
    attn, gdn = first[FULL].attention, first[LINEAR].attention
    if isinstance(first[LINEAR], ReorderedNormTransformerBlock):
        log.warning("The Gated DeltaNet blocks are post-norm but olmo_hybrid applies pre-norm to linear_attention layers; "
                    "the exported model's outputs may differ")
    config: Dict[str, Any] = {
        "model_type": "olmo_hybrid",
        "architectures": ["OlmoHybridForCausalLM"],
        "vocab_size": model.vocab_size,
        "hidden_size": model.d_model,
        "intermediate_size": first[FULL].feed_forward.hidden_size,
        "num_hidden_layers": len(layer_types),
        "num_attention_heads": attn.n_heads,
        "num_key_value_heads": attn.n_kv_heads,
        "hidden_act": "silu",
        "max_position_embeddings": max_seq_len,
        "initializer_range": 0.02,
        "use_cache": True,
        "attention_bias": attn.w_out.bias is not None,
        "attention_dropout": 0.0,
        "rms_norm_eps": first[FULL].feed_forward_norm.eps,
        "tie_word_embeddings": getattr(model, "tie_word_embeddings", False),
        "layer_types": list(layer_types),
        "linear_num_key_heads": gdn.n_heads,
        "linear_num_value_heads": gdn.n_v_heads,
        "linear_key_head_dim": gdn.head_k_dim,
        "linear_value_head_dim": gdn.head_v_dim,
        "linear_conv_kernel_dim": gdn.conv_size,
        "linear_allow_neg_eigval": gdn.allow_neg_eigval,
        "pad_token_id": None,  # the token ids are filled in once a tokenizer is saved next to the model
        "bos_token_id": None,
        "eos_token_id": None,
    }
    rope = _rope_parameters(model, layer_types)
    if rope is not None:
        config["rope_parameters"] = rope
    else:
        config["rope_theta"] = None
    return config


def convert_hybrid_state_to_hf(state_dict: Dict[str, Any], layer_types: List[str]) -> Dict[str, Any]:
    """An unsharded state dict of a hybrid model under its ``olmo_hybrid`` names. Unknown keys raise ``KeyError``."""
    out: Dict[str, Any] = {}
    for key, value in state_dict.items():
        if key in _TOP_LEVEL:
            out[_TOP_LEVEL[key]] = value
            continue
        m = _BLOCK_KEY.match(key)
        if m is None:
            raise KeyError(f"Unmapped key: {key}")
        layer, rest = int(m.group(1)), m.group(2)
        table = _LAYER_TABLES[layer_types[layer]]
        if rest not in table:
            raise KeyError(f"Unmapped block suffix for layer {layer} (type={layer_types[layer]!r}): {key}")
        out[f"model.layers.{layer}.{table[rest]}"] = value
    return out


def save_hf_hybrid_model(save_dir: PathOrStr, model_state_dict: Dict[str, Any], model, *, dtype: Optional[DType] = None,
                         vocab_size: Optional[int] = None, max_sequence_length: int = 65536) -> None:
    """
    Write a hybrid model as ``config.json`` + ``model.safetensors`` under ``save_dir``. ``dtype`` casts the weights,
    ``vocab_size`` cuts the embedding and output rows (padding rows added for training are dropped).
    """
    from safetensors.torch import save_file

    from ...distributed.utils import get_full_tensor

    layer_types = get_hybrid_layer_types(model)
    config = get_hybrid_hf_config(model, layer_types, max_seq_len=max_sequence_length)
    state = convert_hybrid_state_to_hf({k: get_full_tensor(v) for k, v in model_state_dict.items()}, layer_types)
    if dtype is not None:
        state = {k: v.to(DType(dtype).as_pt()) if torch.is_tensor(v) else v for k, v in state.items()}
    if vocab_size is not None:
        config["vocab_size"] = vocab_size
        for name in ("model.embed_tokens.weight", "lm_head.weight"):
            if name in state:
                state[name] = state[name][:vocab_size]
    state = {k: v.contiguous() for k, v in state.items()}
    path = Path(save_dir)
    path.mkdir(parents=True, exist_ok=True)
    with open(path / "config.json", "w") as f:
        json.dump(config, f, indent=2)
    save_file(state, str(path / "model.safetensors"))
    log.info(f"Saved {len(state)} tensors and config.json to {path}")


# ---------------------------------------------------------------------------------------------------------------
# Qwen3.5 (Gated DeltaNet + gated full attention) -> this framework
# ---------------------------------------------------------------------------------------------------------------

_OFFSET_NORMS = ("attention_norm.weight", "feed_forward_norm.weight", "lm_head.norm.weight", "q_norm.weight", "k_norm.weight")


def _text_decoder_state(hf_state: Dict[str, Any]) -> Dict[str, Any]:
    """
    The text decoder's tensors under plain ``model.layers.*`` / ``model.embed_tokens`` / ``model.norm`` / ``lm_head``
    names: multimodal checkpoints nest the decoder (``model.language_model.*``) and carry a vision tower, which is
    dropped.
    """
    out: Dict[str, Any] = {}
    for key, value in hf_state.items():
        if any(part in key for part in ("visual.", "vision_tower", "multi_modal")):
            continue
        if ".layers." in key:
            out["model" + key[key.index(".layers."):]] = value
        elif key.endswith("embed_tokens.weight"):
            out["model.embed_tokens.weight"] = value
        elif key.endswith("norm.weight"):
            out["model.norm.weight"] = value
        elif key == "lm_head.weight" or key.endswith(".lm_head.weight"):
            out["lm_head.weight"] = value
    return out


def _first(state: Dict[str, Any], *names: str):
    for n in names:
        if n in state:
            return state[n]
    raise KeyError(names[0])


def convert_qwen3_5_state_from_hf(config, hf_state: Dict[str, Any]) -> Dict[str, Any]:
    """
    A Hugging Face Qwen3.5 text-model state dict under this framework's names. Differences that a name table cannot
    express: the Gated DeltaNet q/k/v projections and their convolutions are fused (split by rows into ``key_dim``,
    ``key_dim``, ``value_dim``); the attention query projection carries the output gate interleaved per head
    (``[q_0, g_0, q_1, g_1, ...]`` -> ``w_q``, ``w_g``); and the RMSNorm weights are stored as offsets from one.
    """
    cfg = getattr(config, "text_config", None) or config
    src = _text_decoder_state(hf_state)
    key_dim = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    value_dim = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    out: Dict[str, Any] = {}
    if "model.embed_tokens.weight" in src:
        out["embeddings.weight"] = src["model.embed_tokens.weight"]
    if "model.norm.weight" in src:
        out["lm_head.norm.weight"] = src["model.norm.weight"]
    if "lm_head.weight" in src:
        out["lm_head.w_out.weight"] = src["lm_head.weight"]
    elif getattr(cfg, "tie_word_embeddings", False) and "model.embed_tokens.weight" in src:
        out["lm_head.w_out.weight"] = src["model.embed_tokens.weight"]

    for i, kind in enumerate(list(cfg.layer_types)[: cfg.num_hidden_layers]):
        hf, ours = f"model.layers.{i}.", f"blocks.{i}."
        if kind == LINEAR:
            la = hf + "linear_attn."
            cuts = [key_dim, key_dim, value_dim]
            for name, w in zip("qkv", torch.split(src[la + "in_proj_qkv.weight"][: 2 * key_dim + value_dim], cuts)):
                out[f"{ours}attention.w_{name}.weight"] = w
            for name, w in zip("qkv", torch.split(src[la + "conv1d.weight"][: 2 * key_dim + value_dim], cuts)):
                out[f"{ours}attention.{name}_conv1d.weight"] = w
            out[ours + "attention.w_g.weight"] = src[la + "in_proj_z.weight"]
            out[ours + "attention.w_a.weight"] = src[la + "in_proj_a.weight"]
            out[ours + "attention.w_b.weight"] = src[la + "in_proj_b.weight"]
            out[ours + "attention.w_out.weight"] = _first(src, la + "o_proj.weight", la + "out_proj.weight")
            out[ours + "attention.o_norm.weight"] = _first(src, la + "o_norm.weight", la + "norm.weight")
            out[ours + "attention.A_log"] = src[la + "A_log"]
            out[ours + "attention.dt_bias"] = src[la + "dt_bias"]
        elif kind == FULL:
            sa = hf + "self_attn."
            fused = src[sa + "q_proj.weight"]
            per_head = fused.view(cfg.num_attention_heads, 2, cfg.head_dim, fused.shape[1])
            out[ours + "attention.w_q.weight"] = per_head[:, 0].reshape(-1, fused.shape[1])
            out[ours + "attention.w_g.weight"] = per_head[:, 1].reshape(-1, fused.shape[1])
            for name, theirs in (("w_k", "k_proj"), ("w_v", "v_proj"), ("w_out", "o_proj"), ("q_norm", "q_norm"),
                                 ("k_norm", "k_norm")):
                out[f"{ours}attention.{name}.weight"] = src[f"{sa}{theirs}.weight"]
        else:
            raise ValueError(f"Unknown layer type {kind!r} at layer {i}")
        out[ours + "attention_norm.weight"] = src[hf + "input_layernorm.weight"]
        out[ours + "feed_forward_norm.weight"] = src[hf + "post_attention_layernorm.weight"]
        for mine, theirs in _MLP.items():
            out[ours + mine] = src[hf + theirs]

    # Qwen3.5 applies ``x * (1 + weight)`` with zero-initialised weights; this framework applies ``x * weight``
    for key, value in out.items():
        if torch.is_tensor(value) and any(p in key for p in _OFFSET_NORMS):
            out[key] = value + 1.0
    return out
