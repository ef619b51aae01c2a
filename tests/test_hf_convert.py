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
