"""Smaller API modules: state conversion templates, fs cache, launch configs, experiment / ladder CLIs, vision, chat, fp8 emulation."""

import os
import sys

import pytest
import torch


def test_state_converter_templates():
    from olmo_core_b200.nn.conversion import StateConverter, StateMappingTemplate, TemplatePlaceholder

    conv = StateConverter([
        StateMappingTemplate("blocks.[layer].w", "model.layers.[layer].w"),
        StateMappingTemplate(("blocks.[layer].q", "blocks.[layer].k"), "model.layers.[layer].qk", source_concat_dim=0),
        StateMappingTemplate("blocks.[layer].experts.w1", "model.layers.[layer].experts.[expert].gate.weight",
                             dest_key_per_placeholder=TemplatePlaceholder.EXPERT,
                             unflatten_dim=(0, (TemplatePlaceholder.EXPERT, -1)), dims_permutation=(0, 2, 1),
                             flatten_dims=(0, 1)),
    ])
    state = {"blocks.0.w": torch.ones(2), "blocks.1.w": torch.zeros(2), "blocks.0.q": torch.ones(2, 3),
             "blocks.0.k": torch.zeros(1, 3), "blocks.1.experts.w1": torch.arange(24.0).view(12, 2)}
    out = conv.convert(state, {TemplatePlaceholder.LAYER: 2, TemplatePlaceholder.EXPERT: 4})
    assert out["model.layers.0.qk"].shape == (3, 3)
    assert out["model.layers.1.experts.2.gate.weight"].shape == (2, 3)
    torch.testing.assert_close(out["model.layers.1.experts.0.gate.weight"], torch.arange(6.0).view(3, 2).t())
    with pytest.raises(RuntimeError):
        conv.convert({"unknown": torch.ones(1)}, {TemplatePlaceholder.LAYER: 1})


def test_fs_cache(tmp_path, monkeypatch):
    from olmo_core_b200.fs_cache import CACHE_DIR_ENV_VAR, maybe_cache

    calls = []

    @maybe_cache(condition=lambda a, b=1: a >= 0)
    def add(a, b=1):
        calls.append((a, b))
        return a + b

    assert add(1, b=2) == 3 and add(1, b=2) == 3 and len(calls) == 2  # no cache dir: plain calls
    monkeypatch.setenv(CACHE_DIR_ENV_VAR, str(tmp_path))
    assert add(1, b=2) == 3 and add(1, b=2) == 3 and len(calls) == 3  # second call served from disk
    assert add(-1) == 0 and add(-1) == 0 and len(calls) == 5  # the condition vetoes caching
    assert len(list(tmp_path.glob("*.pkl"))) == 1


def test_launch_configs():
    from olmo_core_b200.launch.beaker import BeakerEnvVar, BeakerLaunchConfig, is_running_in_beaker
    from olmo_core_b200.launch.local import LocalLaunchConfig
    from olmo_core_b200.launch.utils import parse_git_remote_url

    assert parse_git_remote_url("git@github.com:allenai/OLMo-core.git") == ("allenai", "OLMo-core")
    assert parse_git_remote_url("https://github.com/allenai/OLMo-core") == ("allenai", "OLMo-core")
    with pytest.raises(ValueError):
        parse_git_remote_url("https://gitlab.com/a/b")
    assert not is_running_in_beaker()
    cfg = BeakerLaunchConfig(name="run", cmd=["train.py", "x=1"], num_nodes=2, git=None,
                             env_vars=[BeakerEnvVar(name="NCCL_DEBUG", value="WARN")])
    spec = cfg.build_experiment_spec()
    assert spec["command"][0] == "torchrun" and "--nnodes=2:2" in spec["command"] and spec["replicas"] == 2
    assert dict(spec["env_vars"])["NCCL_DEBUG"] == "WARN" and dict(spec["env_vars"])["NUM_NODES"] == "2"
    single = BeakerLaunchConfig(name="run", cmd=["train.py"], num_gpus=1, git=None).build_experiment_spec()
    assert single["command"] == ["python", "train.py"]
    local = LocalLaunchConfig(cmd=["train.py"], num_gpus=4).build_command()
    assert "--nproc-per-node=4" in local and "127.0.0.1" in local


def test_experiment_config_builder(monkeypatch):
    from olmo_core_b200.data import TokenizerConfig
    from olmo_core_b200.internal import cookbook, experiment as ex
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.optim import CosWithWarmup
    from olmo_core_b200.train import Duration

    monkeypatch.setenv("OLMO_CORE_ROOT_DIR", "/tmp/olmo-root")
    ctx = ex.CliContext("s.py", ex.SubCmd.dry_run, "run1", "local", ["--trainer.max_duration.value=5"])
    cfg = ex.build_config(
        ctx, global_batch_size=8 * 4096, tokenizer=TokenizerConfig.gpt2(),
        model_config_builder=lambda c: TransformerConfig.olmo2_30M(vocab_size=c.tokenizer.padded_vocab_size()),
        train_module_config_builder=lambda c: cookbook.configure_train_module(
            c.max_sequence_length, 8192, 3e-4, CosWithWarmup(warmup_steps=10), activation_memory_budget=0.5),
        trainer_config_builder=lambda c: cookbook.configure_trainer(Duration.steps(100), c.save_folder, c.work_dir))
    assert cfg.trainer.max_duration.value == 5  # the override was merged
    assert cfg.trainer.save_folder == "/tmp/olmo-root/checkpoints/run1"
    assert {"config_saver", "garbage_collector", "profiler"} <= set(cfg.trainer.callbacks)
    assert cfg.train_module.ac_config is not None and ctx.remote_cmd[1] == "train"


def test_model_ladder_planning(tmp_path):
    from olmo_core_b200.data import TokenizerConfig
    from olmo_core_b200.model_ladder import (ModelLadder, Olmo3ModelConfigurator, TransformerSize,
                                             WSDSChinchillaRunConfigurator)

    assert TransformerSize("1B") > TransformerSize("760M") and TransformerSize("60M").approx_num_params == 60_000_000
    run = WSDSChinchillaRunConfigurator(chinchilla_multiple=4.0)
    ladder = ModelLadder(name="lad", dir=str(tmp_path), sizes=["60M", "7B"], max_devices=64, device_type="NVIDIA B200",
                         model_configurator=Olmo3ModelConfigurator(), run_configurator=run, data_loader=None,
                         instance_sources=[], tokenizer=TokenizerConfig.dolma2(), sequence_length=4096)
    plan = ladder.dry_run("7B", show_plot=False)
    assert plan["rank_microbatch_size"] == 4 * 4096  # 2 x 4096 on H100, doubled on B200
    assert plan["num_devices"] == 64 and plan["global_batch_size"] % (plan["rank_microbatch_size"] * 64) == 0
    ckpts = run.configure_checkpoint_intervals(60_000_000, 262144)
    assert len(ckpts) == 8 and ckpts[-1][1].endswith("4xC post-decay")  # periods end at 0.5, 1, 2, 4 x Chinchilla
    assert ckpts[-1][0].value == run.configure_duration(60_000_000, 262144).value
    sched = run.configure_lr_scheduler(60_000_000, 262144)
    assert sum(sched.period_lengths) == ckpts[-1][0].value
    infos = ladder.get_checkpoints("60M")
    assert infos[0].name == "initialization" and not any(i.exists for i in infos)
    with pytest.raises(Exception):
        ModelLadder(name="x", dir=str(tmp_path), sizes=["13B"], max_devices=8, device_type="b200",
                    model_configurator=Olmo3ModelConfigurator(), run_configurator=run, data_loader=None,
                    instance_sources=[], tokenizer=TokenizerConfig.dolma2(), sequence_length=4096)


def test_vision_language_model():
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.nn.vision import MultimodalLMConfig, VisionConnectorConfig, VisionEncoderConfig

    torch.manual_seed(0)
    vis = VisionEncoderConfig.siglip_b16_224()
    vis.image_num_layers, vis.image_emb_dim, vis.image_num_heads = 2, 64, 4
    vis.image_num_key_value_heads, vis.image_head_dim, vis.image_mlp_dim = 4, 16, 128
    lm = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2)
    conn = VisionConnectorConfig.from_vision_encoder(vis, output_dim=lm.d_model, num_input_layers=2,
                                                     pooling_attention_mask=True)
    model = MultimodalLMConfig(lm=lm, vision=vis, connector=conn, image_patch_token_id=7, vit_layers=(-1, -2)).build()
    B, crops, patches = 2, 2, 196
    images = torch.randn(B, crops, patches, 16 * 16 * 3)
    idx = torch.randint(0, crops * patches, (B, 5, 4))
    idx[0, 0, 3] = -1
    ids = torch.randint(8, 512, (B, 32))
    ids[:, :5] = 7
    out = model(ids, images=images, pooled_patches_idx=idx)
    text_only = model(ids)
    assert out.shape == (B, 32, 512) and not torch.allclose(out, text_only)
    out.float().sum().backward()
    assert model.vision.patch_embedding.weight.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        model(ids[:, 4:], images=images, pooled_patches_idx=idx)  # one placeholder short
    assert VisionEncoderConfig().build(init_device="meta").num_prefix_tokens == 1


def test_chat_session_commands():
    from olmo_core_b200.generate.chat import ChatSession

    class Tok:
        def apply_chat_template(self, history, **kwargs):
            return "".join(m["content"] for m in history)

        def encode(self, text, return_tensors=None):
            return torch.tensor([[ord(c) for c in text]])

        def decode(self, ids, skip_special_tokens=True):
            return "".join(chr(int(i)) for i in ids)

    class Module:
        def generate_batch(self, ids, **kwargs):
            return ids.flip(1), None, None

    s = ChatSession(Module(), Tok(), system_prompt="S:")
    assert s.handle("abc") == "cba:S" and len(s.history) == 3
    assert s.handle("/clear") and len(s.history) == 1
    assert s.handle("  ") == "" and s.handle("/help").startswith("Commands") and s.handle("/exit") is None


def test_fp8_emulation_error_stays_at_e4m3_level():
    from olmo_core_b200.ops.fp8 import fp8_linear, quantize_colwise_transposed, quantize_rowwise

    torch.manual_seed(0)
    x = torch.randn(64, 128).bfloat16().requires_grad_(True)
    w = (torch.randn(96, 128) * 0.05).bfloat16().requires_grad_(True)
    q, s = quantize_rowwise(x.detach(), pow2=True)
    assert torch.equal(torch.log2(s), torch.log2(s).round())  # scales are powers of two
    qt, st = quantize_colwise_transposed(x.detach())
    assert qt.shape == (128, 64) and st.shape == (128,)
    y = fp8_linear(x, w)
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).norm() / ref.norm()) < 0.06
    y.backward(torch.ones_like(y))
    assert x.grad is not None and w.grad is not None
