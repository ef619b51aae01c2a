"""
Parameter-name (and layout) mapping between this framework's transformer state dicts and Hugging Face causal-LM
state dicts (role of src/olmo_core/nn/hf/convert.py).

The mapping is a table of name templates: ``{layer}`` and ``{expert}`` are expanded over the model's layers / experts.
Dense models map one to one. Mixture-of-experts weights are stored here as stacked ``[E * in, out]`` / ``[E * out, in]``
matrices and on the HF side as one ``nn.Linear`` per expert, so they are split / concatenated (and transposed) on the
way. RoPE uses the same "rotate half" convention on both sides, so projections need no permutation.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

__all__ = ["convert_state_to_hf", "convert_state_from_hf", "fuse_expert_weights", "split_expert_weights", "get_converter_to_hf", "get_converter_from_hf",
           "OLMO_CORE_TO_HF_TEMPLATES", "StateConverter"]

# (this framework, Hugging Face). Norm names depend on the block type, see ``_norm_templates``.
OLMO_CORE_TO_HF_TEMPLATES: List[Tuple[str, str]] = [
    ("embeddings.weight", "model.embed_tokens.weight"),
    ("lm_head.norm.weight", "model.norm.weight"),
    ("lm_head.w_out.weight", "lm_head.weight"),
    ("blocks.{layer}.attention.w_q.weight", "model.layers.{layer}.self_attn.q_proj.weight"),
    ("blocks.{layer}.attention.w_k.weight", "model.layers.{layer}.self_attn.k_proj.weight"),
    ("blocks.{layer}.attention.w_v.weight", "model.layers.{layer}.self_attn.v_proj.weight"),
    ("blocks.{layer}.attention.w_out.weight", "model.layers.{layer}.self_attn.o_proj.weight"),
    ("blocks.{layer}.attention.w_q.bias", "model.layers.{layer}.self_attn.q_proj.bias"),
    ("blocks.{layer}.attention.w_k.bias", "model.layers.{layer}.self_attn.k_proj.bias"),
    ("blocks.{layer}.attention.w_v.bias", "model.layers.{layer}.self_attn.v_proj.bias"),
    ("blocks.{layer}.attention.w_out.bias", "model.layers.{layer}.self_attn.o_proj.bias"),
    ("blocks.{layer}.attention.q_norm.weight", "model.layers.{layer}.self_attn.q_norm.weight"),
    ("blocks.{layer}.attention.k_norm.weight", "model.layers.{layer}.self_attn.k_norm.weight"),
    ("blocks.{layer}.feed_forward.w1.weight", "model.layers.{layer}.mlp.gate_proj.weight"),
    ("blocks.{layer}.feed_forward.w2.weight", "model.layers.{layer}.mlp.down_proj.weight"),
    ("blocks.{layer}.feed_forward.w3.weight", "model.layers.{layer}.mlp.up_proj.weight"),
    ("blocks.{layer}.feed_forward_moe.router.weight", "model.layers.{layer}.mlp.gate.weight"),
]

_MOE_EXPERT_TEMPLATES = [  # (stacked name here, per-expert HF name, transpose when splitting)
    ("blocks.{layer}.feed_forward_moe.experts.mlp.w1", "model.layers.{layer}.mlp.experts.{expert}.gate_proj.weight", True),
    ("blocks.{layer}.feed_forward_moe.experts.mlp.w2", "model.layers.{layer}.mlp.experts.{expert}.down_proj.weight", False),
    ("blocks.{layer}.feed_forward_moe.experts.mlp.w3", "model.layers.{layer}.mlp.experts.{expert}.up_proj.weight", True),
]


def _norm_templates(style: str) -> List[Tuple[str, str]]:
    """Block norms by architecture family (src/olmo_core/nn/hf/convert.py:99-121 lists the same per-model overrides)."""
    if style == "reordered":  # OLMo-2 / OLMo-3 / FlexOlmo: norms are applied to the sub-layer outputs
        return [("blocks.{layer}.attention_norm.weight", "model.layers.{layer}.post_attention_layernorm.weight"),
                ("blocks.{layer}.feed_forward_norm.weight", "model.layers.{layer}.post_feedforward_layernorm.weight")]
    if style == "peri":  # Gemma-3: a norm on the input and on the output of both sub-layers
        return [("blocks.{layer}.attention_norm.weight", "model.layers.{layer}.input_layernorm.weight"),
                ("blocks.{layer}.post_attention_norm.weight", "model.layers.{layer}.post_attention_layernorm.weight"),
                ("blocks.{layer}.feed_forward_norm.weight", "model.layers.{layer}.pre_feedforward_layernorm.weight"),
                ("blocks.{layer}.post_feed_forward_norm.weight", "model.layers.{layer}.post_feedforward_layernorm.weight")]
    # Llama, Qwen-3, OLMoE: norms on the sub-layer inputs
    return [("blocks.{layer}.attention_norm.weight", "model.layers.{layer}.input_layernorm.weight"),
            ("blocks.{layer}.feed_forward_norm.weight", "model.layers.{layer}.post_attention_layernorm.weight")]


_NORM_STYLE_BY_MODEL_TYPE = {"olmo2": "reordered", "olmo3": "reordered", "flex_olmo": "reordered", "gemma3_text": "peri",
                             "gemma3": "peri"}
# Gemma's RMSNorm multiplies by (1 + weight) with zero-initialised weights; every norm here multiplies by its weight.
_UNIT_OFFSET_NORM_MODEL_TYPES = ("gemma3_text", "gemma3")
_NORM_SUFFIXES = ("attention_norm.weight", "post_attention_norm.weight", "feed_forward_norm.weight",
                  "post_feed_forward_norm.weight", "lm_head.norm.weight", "q_norm.weight", "k_norm.weight")


def _shift_norm_weights(state: Dict[str, Any], delta: float) -> Dict[str, Any]:
    return {k: (v + delta if isinstance(v, torch.Tensor) and k.endswith(_NORM_SUFFIXES) else v) for k, v in state.items()}


class StateConverter:
    """Expands the templates for a concrete number of layers / experts and renames (splits, merges) tensors."""

    def __init__(self, n_layers: int, n_experts: int = 0, reordered_norm: bool = True, norm_style: Optional[str] = None):
        self.n_layers, self.n_experts = n_layers, n_experts
        self.pairs: List[Tuple[str, str]] = []
        style = norm_style or ("reordered" if reordered_norm else "pre")
        for ours, theirs in OLMO_CORE_TO_HF_TEMPLATES + _norm_templates(style):
            if "{layer}" in ours:
                self.pairs += [(ours.format(layer=i), theirs.format(layer=i)) for i in range(n_layers)]
            else:
                self.pairs.append((ours, theirs))

    def to_hf(self, state: Dict[str, Any]) -> Dict[str, Any]:
        out = {theirs: state[ours] for ours, theirs in self.pairs if ours in state}
        for i in range(self.n_layers):
            # the router is stored flat here and as [experts, d_model] there
            key = f"model.layers.{i}.mlp.gate.weight"
            if key in out and out[key].dim() == 1 and self.n_experts:
                out[key] = out[key].view(self.n_experts, -1)
        for ours_t, theirs_t, _ in _MOE_EXPERT_TEMPLATES:
            for i in range(self.n_layers):
                ours = ours_t.format(layer=i)
                if ours not in state:
                    continue
                d_model = state["embeddings.weight"].shape[1] if "embeddings.weight" in state else None
                for e, piece in enumerate(state[ours].chunk(self.n_experts, dim=0)):
                    # HF: gate / up are [hidden, d_model], down is [d_model, hidden]. The stacked matrices here are
                    # [E * hidden, d_model] (dropless experts, all three) or [E * d_model, hidden] (w1, w3 of the
                    # fixed-capacity experts): transpose whichever piece is the other way round.
                    want_rows_d_model = "down_proj" in theirs_t
                    rows_are_d_model = d_model is not None and piece.shape[0] == d_model and piece.shape[1] != d_model
                    transpose = rows_are_d_model != want_rows_d_model if piece.shape[0] != piece.shape[1] else False
                    out[theirs_t.format(layer=i, expert=e)] = piece.t().contiguous() if transpose else piece.contiguous()
        return out

    def from_hf(self, hf_state: Dict[str, Any], dropless: bool = True) -> Dict[str, Any]:
        """``dropless``: the target stores all three expert matrices as ``[E * hidden, d_model]`` (else w1 / w3 as
        ``[E * d_model, hidden]``)."""
        out = {ours: hf_state[theirs] for ours, theirs in self.pairs if theirs in hf_state}
        for i in range(self.n_layers):
            key = f"blocks.{i}.feed_forward_moe.router.weight"
            if key in out and out[key].dim() == 2:
                out[key] = out[key].reshape(-1)
        for ours_t, theirs_t, _ in _MOE_EXPERT_TEMPLATES:
            for i in range(self.n_layers):
                names = [theirs_t.format(layer=i, expert=e) for e in range(self.n_experts)]
                if not names or names[0] not in hf_state:
                    continue
                down = "down_proj" in theirs_t
                transpose = down if dropless else not down  # HF: gate/up [hidden, d], down [d, hidden]
                pieces = [hf_state[n].t() if transpose else hf_state[n] for n in names]
                out[ours_t.format(layer=i)] = torch.cat(pieces, dim=0).contiguous()
        return out


def _converter_for(hf_config, n_experts: Optional[int] = None) -> StateConverter:
    model_type = getattr(hf_config, "model_type", "olmo2")
    experts = n_experts if n_experts is not None else int(getattr(hf_config, "num_experts", 0) or 0)
    return StateConverter(hf_config.num_hidden_layers, n_experts=experts,
                          norm_style=_NORM_STYLE_BY_MODEL_TYPE.get(model_type, "pre"))


def get_converter_to_hf(hf_config=None, model_type: Optional[str] = None) -> StateConverter:
    if hf_config is None:
        raise ValueError("an HF config is needed to expand the name templates")
    return _converter_for(hf_config)


def get_converter_from_hf(hf_config=None, model_type: Optional[str] = None) -> StateConverter:
    return get_converter_to_hf(hf_config, model_type)


def fuse_expert_weights(hf_state: Dict[str, Any], n_layers: int, n_experts: int) -> Dict[str, Any]:
    """
    Per-expert ``experts.<e>.{gate,up,down}_proj.weight`` entries (the layout of checkpoints on the hub) -> the stacked
    ``experts.gate_up_proj [E, 2 * hidden, d_model]`` / ``experts.down_proj [E, d_model, hidden]`` parameters that
    ``transformers`` >= 5 models hold in memory.
    """
    out = dict(hf_state)
    for i in range(n_layers):
        base = f"model.layers.{i}.mlp.experts"
        if f"{base}.0.gate_proj.weight" not in out:
            continue
        gate = [out.pop(f"{base}.{e}.gate_proj.weight") for e in range(n_experts)]
        up = [out.pop(f"{base}.{e}.up_proj.weight") for e in range(n_experts)]
        down = [out.pop(f"{base}.{e}.down_proj.weight") for e in range(n_experts)]
        out[f"{base}.gate_up_proj"] = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gate, up)])
        out[f"{base}.down_proj"] = torch.stack(down)
    return out


def split_expert_weights(hf_state: Dict[str, Any], n_layers: int) -> Dict[str, Any]:
    """The inverse of :func:`fuse_expert_weights`."""
    out = dict(hf_state)
    for i in range(n_layers):
        base = f"model.layers.{i}.mlp.experts"
        if f"{base}.gate_up_proj" not in out:
            continue
        gate_up, down = out.pop(f"{base}.gate_up_proj"), out.pop(f"{base}.down_proj")
        hidden = gate_up.shape[1] // 2
        for e in range(gate_up.shape[0]):
            out[f"{base}.{e}.gate_proj.weight"] = gate_up[e, :hidden]
            out[f"{base}.{e}.up_proj.weight"] = gate_up[e, hidden:]
            out[f"{base}.{e}.down_proj.weight"] = down[e]
    return out


def convert_state_to_hf(config, olmo_core_state: Dict[str, Any], fused_experts: bool = False) -> Dict[str, Any]:
    """State dict of this framework's transformer -> state dict of the HF causal LM described by the HF ``config``
    (``fused_experts``: stacked expert parameters as ``transformers`` >= 5 models expect them in memory)."""
    hf_config, state = config, olmo_core_state
    if getattr(hf_config, "model_type", None) in _UNIT_OFFSET_NORM_MODEL_TYPES:
        state = _shift_norm_weights(state, -1.0)
    converted = _converter_for(hf_config).to_hf(state)
    if fused_experts:
        converted = fuse_expert_weights(converted, hf_config.num_hidden_layers, int(getattr(hf_config, "num_experts", 0) or 0))
    if getattr(hf_config, "tie_word_embeddings", False):
        converted.pop("lm_head.weight", None)
    missing = [k for k in state if not any(k == ours for ours, _ in _converter_for(hf_config).pairs)
               and "experts.mlp" not in k and not k.endswith(("router.score_bias", "batch_size_per_expert"))]
    if missing:
        raise KeyError(f"no Hugging Face counterpart for parameters: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    return converted


def convert_state_from_hf(config, hf_state: Dict[str, Any], model_type: Optional[str] = None) -> Dict[str, Any]:
    """State dict of the HF causal LM described by the HF ``config`` -> state dict of this framework's transformer."""
    hf_config = config
    hf_state = split_expert_weights(hf_state, hf_config.num_hidden_layers)
    converted = _converter_for(hf_config).from_hf(hf_state)
    if getattr(hf_config, "model_type", None) in _UNIT_OFFSET_NORM_MODEL_TYPES:
        converted = _shift_norm_weights(converted, 1.0)
    if "lm_head.w_out.weight" not in converted and "embeddings.weight" in converted:
        converted["lm_head.w_out.weight"] = converted["embeddings.weight"]  # tied embeddings
    return converted


def __getattr__(name: str):
    # defined in ``hybrid.py``; reachable under this module's name as well
    if name in ('convert_hybrid_state_to_hf', 'convert_qwen3_5_state_from_hf'):
        from . import hybrid

        return getattr(hybrid, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
