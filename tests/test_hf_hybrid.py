"""Hybrid (Gated DeltaNet + attention) models: ``olmo_hybrid`` export names and config, Qwen3.5 state import."""

import json
from types import SimpleNamespace

import pytest
import torch

from olmo_core_b200.nn.hf import (
    convert_hybrid_state_to_hf,
    convert_qwen3_5_state_from_hf,
    get_hybrid_hf_config,
    get_hybrid_layer_types,
    is_olmo_hybrid_model,
    save_hf_hybrid_model,
)
from olmo_core_b200.nn.transformer import TransformerConfig


def _hybrid(gate: bool):
    cfg = TransformerConfig.qwen3_5_like(
        d_model=64, vocab_size=128, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=16, intermediate_size=96,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=16,
        tie_word_embeddings=False)
    if not gate:
        cfg.block["attn"].sequence_mixer.gate = None
    torch.manual_seed(0)
    model = cfg.build(init_device="cpu")
    model.init_weights(max_seq_len=32, device=torch.device("cpu"))
    return model


def test_hybrid_export_names_config_and_files(tmp_path):
    pytest.importorskip("safetensors")
    from safetensors.torch import load_file

    model = _hybrid(gate=False)
    assert is_olmo_hybrid_model(model)
    assert not is_olmo_hybrid_model(TransformerConfig.olmo2_30M(vocab_size=64, n_layers=1).build(init_device="meta"))
    types = get_hybrid_layer_types(model)
    assert types == ["linear_attention"] * 3 + ["full_attention"]
    state = model.state_dict()
    hf = convert_hybrid_state_to_hf(state, types)
    assert len(hf) == len(state)
    assert hf["model.layers.0.linear_attn.A_log"] is state["blocks.0.attention.A_log"]
    assert hf["model.layers.0.input_layernorm.weight"] is state["blocks.0.attention_norm.weight"]
    assert hf["model.layers.3.post_attention_layernorm.weight"] is state["blocks.3.attention_norm.weight"]
    assert hf["model.layers.3.self_attn.o_proj.weight"] is state["blocks.3.attention.w_out.weight"]
    assert hf["lm_head.weight"] is state["lm_head.w_out.weight"]
    with pytest.raises(KeyError):
        convert_hybrid_state_to_hf({"blocks.0.attention.unknown": torch.zeros(1)}, types)

    cfg = get_hybrid_hf_config(model, types, max_seq_len=4096)
    assert cfg["model_type"] == "olmo_hybrid" and cfg["layer_types"] == types and cfg["max_position_embeddings"] == 4096
    assert (cfg["linear_num_key_heads"], cfg["linear_num_value_heads"]) == (2, 4)
    assert (cfg["linear_key_head_dim"], cfg["linear_value_head_dim"], cfg["linear_conv_kernel_dim"]) == (8, 16, 4)
    assert cfg["num_attention_heads"] == 4 and cfg["num_key_value_heads"] == 2 and cfg["intermediate_size"] == 96
    assert cfg["rope_parameters"]["rope_type"] == "default"

    save_hf_hybrid_model(tmp_path / "out", state, model, vocab_size=100, max_sequence_length=2048)
    saved_cfg = json.loads((tmp_path / "out" / "config.json").read_text())
    assert saved_cfg["vocab_size"] == 100 and saved_cfg["max_position_embeddings"] == 2048
    saved = load_file(str(tmp_path / "out" / "model.safetensors"))
    assert saved["model.embed_tokens.weight"].shape[0] == 100 and saved["lm_head.weight"].shape[0] == 100
    torch.testing.assert_close(saved["model.layers.1.linear_attn.q_proj.weight"], state["blocks.1.attention.w_q.weight"])


def test_qwen3_5_import_undoes_the_fused_layouts():
    model = _hybrid(gate=True)
    state = model.state_dict()
    types = get_hybrid_layer_types(model)
    n_heads, head_dim = 4, 16
    norms = ("attention_norm.weight", "feed_forward_norm.weight", "lm_head.norm.weight", "q_norm.weight", "k_norm.weight")
    off = {k: (v - 1.0 if any(n in k for n in norms) else v) for k, v in state.items()}  # stored as offsets from one
    # a multimodal-style checkpoint: decoder nested under `model.language_model`, plus a vision tensor to be ignored
    hf = {"model.language_model.embed_tokens.weight": off["embeddings.weight"],
          "model.language_model.norm.weight": off["lm_head.norm.weight"], "lm_head.weight": off["lm_head.w_out.weight"],
          "model.visual.patch_embed.weight": torch.zeros(3)}
    for i, kind in enumerate(types):
        o, h = f"blocks.{i}.", f"model.language_model.layers.{i}."
        if kind == "linear_attention":
            hf[h + "linear_attn.in_proj_qkv.weight"] = torch.cat([off[o + f"attention.w_{n}.weight"] for n in "qkv"])
            hf[h + "linear_attn.conv1d.weight"] = torch.cat([off[o + f"attention.{n}_conv1d.weight"] for n in "qkv"])
            for ours, theirs in (("w_g", "in_proj_z"), ("w_a", "in_proj_a"), ("w_b", "in_proj_b"), ("w_out", "out_proj"),
                                 ("o_norm", "norm")):
                hf[h + f"linear_attn.{theirs}.weight"] = off[o + f"attention.{ours}.weight"]
            hf[h + "linear_attn.A_log"] = off[o + "attention.A_log"]
            hf[h + "linear_attn.dt_bias"] = off[o + "attention.dt_bias"]
        else:
            q = off[o + "attention.w_q.weight"].view(n_heads, 1, head_dim, -1)
            g = off[o + "attention.w_g.weight"].view(n_heads, 1, head_dim, -1)
            hf[h + "self_attn.q_proj.weight"] = torch.cat([q, g], dim=1).reshape(2 * n_heads * head_dim, -1)
            for ours, theirs in (("w_k", "k_proj"), ("w_v", "v_proj"), ("w_out", "o_proj"), ("q_norm", "q_norm"),
                                 ("k_norm", "k_norm")):
                hf[h + f"self_attn.{theirs}.weight"] = off[o + f"attention.{ours}.weight"]
        hf[h + "input_layernorm.weight"] = off[o + "attention_norm.weight"]
        hf[h + "post_attention_layernorm.weight"] = off[o + "feed_forward_norm.weight"]
        for ours, theirs in (("w1", "gate_proj"), ("w2", "down_proj"), ("w3", "up_proj")):
            hf[h + f"mlp.{theirs}.weight"] = off[o + f"feed_forward.{ours}.weight"]
    text = SimpleNamespace(layer_types=types, num_hidden_layers=4, linear_num_key_heads=2, linear_key_head_dim=8,
                           linear_num_value_heads=4, linear_value_head_dim=16, head_dim=head_dim,
                           num_attention_heads=n_heads, tie_word_embeddings=False)
    back = convert_qwen3_5_state_from_hf(SimpleNamespace(text_config=text), hf)
    assert set(back) == set(state)
    for k, v in state.items():
        torch.testing.assert_close(back[k], v, msg=k)
    model.load_state_dict(back)
