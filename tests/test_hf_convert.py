"""Export to Hugging Face format reproduces the logits (OLMo-2 style and Llama style blocks), and imports back."""

import pytest
import torch

transformers = pytest.importorskip("transformers")

from olmo_core_b200.nn.hf import convert_state_from_hf, get_hf_config, save_hf_model, validate_conversion  # noqa: E402
from olmo_core_b200.nn.transformer import TransformerConfig  # noqa: E402


@pytest.mark.parametrize("family", ["olmo2_30M", "llama2_271M"])
def test_export_reproduces_logits(tmp_path, family):
    torch.manual_seed(0)
    kwargs = dict(vocab_size=256, n_layers=2)
    model = getattr(TransformerConfig, family)(**kwargs).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    cfg = get_hf_config(model)
    assert cfg.model_type == ("olmo2" if family.startswith("olmo2") else "llama")
    save_hf_model(tmp_path / "hf", model.state_dict(), model)
    validate_conversion(tmp_path / "hf", model, 256, rtol=1e-4, atol=1e-4)
    hf_model = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "hf"))
    back = convert_state_from_hf(hf_model.config, hf_model.state_dict())
    for name, p in model.state_dict().items():
        torch.testing.assert_close(back[name], p, msg=name)


def test_moe_model_exports_to_flex_olmo_and_matches():
    """A reordered-norm mixture-of-experts model becomes a Hugging Face FlexOlmo model with the same logits."""
    import torch
    from transformers import FlexOlmoForCausalLM

    from olmo_core_b200.nn.hf.config import get_hf_config
    from olmo_core_b200.nn.hf.convert import convert_state_from_hf, convert_state_to_hf
    from olmo_core_b200.nn.transformer import TransformerConfig

    torch.manual_seed(0)
    cfg = TransformerConfig.olmoe_1B_7B(vocab_size=128, n_layers=2)
    cfg.d_model = 64
    cfg.block.sequence_mixer.n_heads = 4
    moe = cfg.block.feed_forward_moe
    moe.num_experts, moe.hidden_size = 8, 48
    moe.router.top_k = 2
    model = cfg.build(init_device="cpu")
    model.init_weights(max_seq_len=32, device=torch.device("cpu"))
    model.eval()
    hf_config = get_hf_config(model)
    assert type(hf_config).__name__ == "FlexOlmoConfig" and hf_config.num_experts == 8 and hf_config.num_experts_per_tok == 2
    hf_state = convert_state_to_hf(hf_config, model.state_dict())
    assert hf_state["model.layers.0.mlp.experts.3.gate_proj.weight"].shape == (48, 64)
    assert hf_state["model.layers.0.mlp.experts.3.down_proj.weight"].shape == (64, 48)
    assert hf_state["model.layers.0.mlp.gate.weight"].shape == (8, 64)
    hf_config.max_position_embeddings = 64
    hf = FlexOlmoForCausalLM(hf_config).eval()
    if any(k.endswith("experts.gate_up_proj") for k in hf.state_dict()):  # transformers >= 5 holds the experts stacked
        hf_state = convert_state_to_hf(hf_config, model.state_dict(), fused_experts=True)
        assert hf_state["model.layers.0.mlp.experts.gate_up_proj"].shape == (8, 96, 64)
    missing, unexpected = hf.load_state_dict(hf_state, strict=False)
    assert not unexpected and all("rotary" in k or "inv_freq" in k for k in missing), (missing, unexpected)
    ids = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        ours = model(ids)
        theirs = hf(ids).logits
    torch.testing.assert_close(ours.float(), theirs.float(), rtol=1e-4, atol=1e-4)
    # and back
    back = convert_state_from_hf(hf_config, hf.state_dict())
    for k, v in model.state_dict().items():
        if k in back:
            assert torch.equal(back[k].reshape(v.shape), v), k


def _tiny_like(hf_config, kind: str):
    """This framework's model with the dimensions of a small Hugging Face config."""
    common = dict(d_model=hf_config.hidden_size, vocab_size=hf_config.vocab_size, n_layers=hf_config.num_hidden_layers,
                  n_heads=hf_config.num_attention_heads, n_kv_heads=hf_config.num_key_value_heads)
    if kind == "gemma3":
        cfg = TransformerConfig.gemma3_like(**common, hidden_size=hf_config.intermediate_size, head_dim=hf_config.head_dim,
                                            local_window_size=hf_config.sliding_window, layer_norm_eps=hf_config.rms_norm_eps)
    else:
        cfg = TransformerConfig.qwen3_0_6B(vocab_size=hf_config.vocab_size, n_layers=hf_config.num_hidden_layers)
        cfg.d_model = hf_config.hidden_size
        mixer = cfg.block.sequence_mixer
        mixer.n_heads, mixer.n_kv_heads, mixer.head_dim = hf_config.num_attention_heads, hf_config.num_key_value_heads, hf_config.head_dim
        mixer.rope.theta = int(hf_config.rope_parameters["rope_theta"])
        cfg.block.feed_forward.hidden_size = hf_config.intermediate_size
        cfg.tie_word_embeddings = bool(hf_config.tie_word_embeddings)
    return cfg


@pytest.mark.parametrize("kind", ["qwen3", "gemma3"])
def test_import_and_export_of_qwen3_and_gemma3(kind):
    """Weights of a Hugging Face Qwen-3 / Gemma-3 text model load into the matching architecture here with the same
    logits (per-head query / key norms; Gemma's four norms per block and its (1 + weight) norm convention), and export
    back to the same tensors and an equivalent config."""
    from olmo_core_b200.nn.hf.convert import convert_state_to_hf

    torch.manual_seed(0)
    if kind == "qwen3":
        hf_config = transformers.Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                             num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                             max_position_embeddings=64, tie_word_embeddings=False)
        hf = transformers.Qwen3ForCausalLM(hf_config).eval()
    else:
        hf_config = transformers.Gemma3TextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=6,
                                                  num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                                  max_position_embeddings=64, sliding_window=8, query_pre_attn_scalar=32)
        hf = transformers.Gemma3ForCausalLM(hf_config).eval()
    with torch.no_grad():  # norm weights away from their initial values, so that a missing (1 + w) shift would show
        for name, p in hf.named_parameters():
            if "norm" in name:
                p.add_(torch.randn_like(p) * 0.1)
    model = _tiny_like(hf_config, kind).build(init_device="cpu")
    model.init_weights(max_seq_len=64, device=torch.device("cpu"))
    model.eval()
    state = convert_state_from_hf(hf_config, hf.state_dict())
    missing, unexpected = model.load_state_dict(state, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        want = hf(ids).logits
        got = model(ids)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)

    exported_cfg = get_hf_config(model)
    assert exported_cfg.model_type == hf_config.model_type
    for field in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim"):
        assert getattr(exported_cfg, field) == getattr(hf_config, field), field
    if kind == "gemma3":
        assert exported_cfg.layer_types == hf_config.layer_types and exported_cfg.sliding_window == 8
    back = convert_state_to_hf(exported_cfg, model.state_dict())
    for name, p in hf.state_dict().items():
        if name == "lm_head.weight" and name not in back:
            continue  # tied to the embeddings
        torch.testing.assert_close(back[name], p, msg=name)
