"""Checkpoint utilities (merging of framework and Hugging Face checkpoints) and the HF export callback."""

import json
from pathlib import Path

import pytest
import torch


def test_merge_checkpoints_averages_model_weights(tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_keys, save_state_dict
    from olmo_core_b200.scripts.merge_checkpoints import main, merge

    torch.manual_seed(0)
    states = []
    for i in range(3):
        state = {"blocks.0.w": torch.randn(4, 6), "lm_head.w_out.weight": torch.randn(8, 4).bfloat16()}
        save_state_dict(str(tmp_path / f"step{i}" / "model_and_optim"), {"model": state, "optim": {"step": torch.tensor(i)}})
        states.append(state)
    out = tmp_path / "soup"
    merge(str(out), [str(tmp_path / f"step{i}") for i in range(3)], weights=[0.5, 0.25, 0.25])
    w, head = load_keys(str(out / "model_and_optim"), ["model.blocks.0.w", "model.lm_head.w_out.weight"])
    want = 0.5 * states[0]["blocks.0.w"] + 0.25 * states[1]["blocks.0.w"] + 0.25 * states[2]["blocks.0.w"]
    torch.testing.assert_close(w, want)
    assert head.dtype == torch.bfloat16  # written back in the dtype it had
    want_head = sum(s["lm_head.w_out.weight"].float() for s in states[:2]) / 2
    with pytest.raises(ValueError):
        merge(str(tmp_path / "bad"), [str(tmp_path / "step0"), str(tmp_path / "step1")], weights=[0.9, 0.9])
    # command line, equal weights over the first two
    main([str(tmp_path / "soup2"), str(tmp_path / "step0"), str(tmp_path / "step1")])
    (head2,) = load_keys(str(tmp_path / "soup2" / "model_and_optim"), ["model.lm_head.w_out.weight"])
    torch.testing.assert_close(head2.float(), want_head.bfloat16().float())


def test_merge_hf_checkpoints_averages_floating_point_tensors(tmp_path):
    transformers = pytest.importorskip("transformers")
    from olmo_core_b200.scripts.merge_hf_checkpoints import main

    config = transformers.Olmo2Config(vocab_size=64, hidden_size=16, intermediate_size=32, num_hidden_layers=1,
                                      num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=32)
    dirs, models = [], []
    for i in range(2):
        torch.manual_seed(10 + i)
        model = transformers.AutoModelForCausalLM.from_config(config)
        path = tmp_path / f"hf{i}"
        model.save_pretrained(path)
        dirs.append(str(path))
        models.append(model)
    out = tmp_path / "merged"
    main([*dirs, "--output", str(out), "--weights", "0.75", "0.25"])
    merged = transformers.AutoModelForCausalLM.from_pretrained(out)
    a, b, m = models[0].state_dict(), models[1].state_dict(), merged.state_dict()
    assert set(m) == set(a)
    for key, value in m.items():
        if value.is_floating_point():
            torch.testing.assert_close(value, 0.75 * a[key] + 0.25 * b[key], msg=key)
    assert json.loads((out / "config.json").read_text())["hidden_size"] == 16


def test_hf_converter_callback_exports_the_last_checkpoint(tmp_path):
    pytest.importorskip("transformers")
    from test_trainer import VOCAB, _build  # same folder

    from olmo_core_b200.config import DType
    from olmo_core_b200.train.callbacks import ConfigSaverCallback, HFConverterCallback

    trainer, _ = _build(tmp_path, max_steps=2, save_interval=2)
    saver = ConfigSaverCallback()
    saver.config = {"model": trainer.train_module.model_config_dict() if hasattr(trainer.train_module, "model_config_dict")
                    else None, "dataset": {"tokenizer": {"vocab_size": VOCAB, "eos_token_id": 1, "pad_token_id": 0}}}
    if saver.config["model"] is None:
        from olmo_core_b200.nn.transformer import TransformerConfig

        saver.config["model"] = TransformerConfig.olmo2_30M(vocab_size=VOCAB, n_layers=2).as_config_dict()
    trainer.add_callback("config_saver", saver)
    out = tmp_path / "exported"
    trainer.add_callback("hf", HFConverterCallback(output_folder=str(out), dtype=DType.float32, validate=True,
                                                   max_sequence_length=32))
    trainer.fit()
    assert (out / "config.json").is_file() and any(p.suffix == ".safetensors" for p in out.iterdir())
    import transformers

    hf = transformers.AutoModelForCausalLM.from_pretrained(out)
    ids = torch.randint(0, VOCAB, (1, 16))
    with torch.no_grad():
        want = trainer.train_module.model(ids)
        got = hf(ids).logits
    torch.testing.assert_close(got[..., :VOCAB], want[..., :VOCAB].float(), rtol=1e-3, atol=1e-3)
