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
