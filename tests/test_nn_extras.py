"""Smaller nn pieces: output-discarding checkpoint, causal convolution, gated delta rule, CE module (CPU)."""

import torch
import torch.nn.functional as F

from olmo_core_b200.nn.attention.recurrent import GatedDeltaNetConfig, gated_delta_rule, gated_delta_rule_recurrent
from olmo_core_b200.nn.convolution import CausalConv1d
from olmo_core_b200.nn.cross_entropy_loss import CrossEntropyLoss
from olmo_core_b200.nn.output_discard_checkpoint import OutputDiscardCheckpoint


def test_output_discard_checkpoint_matches_plain_autograd():
    torch.manual_seed(0)
    w1, w2 = torch.randn(8, 16, requires_grad=True), torch.randn(16, 4, requires_grad=True)
    x = torch.randn(5, 8, requires_grad=True)

    def fn(inp, w):
        return F.gelu(inp @ w)

    ref = (fn(x, w1) @ w2).pow(2).sum()
    ref_grads = torch.autograd.grad(ref, (x, w1, w2))

    ckpt = OutputDiscardCheckpoint()
    h = ckpt.checkpoint(fn, x, w1)
    y = h @ w2
    ckpt.discard_output_and_register_recompute(y)
    assert h.untyped_storage().size() == 0  # the intermediate really is gone between forward and backward
    loss = y.pow(2).sum()
    grads = torch.autograd.grad(loss, (x, w1, w2))
    torch.testing.assert_close(loss, ref)
    for a, b in zip(grads, ref_grads):
        torch.testing.assert_close(a, b)


def test_native_storage_rebind_is_zero_copy_and_reaches_saved_views():
    from olmo_core_b200.nn.output_discard_checkpoint import native_rebind_available
    from olmo_core_b200.ops.build import build_native

    build_native(verbose=False)
    assert native_rebind_available()
    kept = torch.arange(12.0)
    view = kept.view(3, 4)  # stands for an autograd-saved alias of the discarded tensor
    impl = kept.untyped_storage()._cdata
    kept.untyped_storage().resize_(0)
    fresh = torch.full((12,), 7.0)
    fresh_ptr = fresh.data_ptr()
    torch.ops.ocb_native.rebind_storage(kept, fresh)
    assert kept.untyped_storage()._cdata == impl and kept.data_ptr() == fresh_ptr and kept._version == 0
    del fresh  # the borrowed allocation stays alive through the reference the rebound storage holds
    assert torch.equal(view, torch.full((3, 4), 7.0))


def test_causal_conv_is_causal_and_respects_documents():
    torch.manual_seed(0)
    conv = CausalConv1d(hidden_size=6, kernel_size=4, activation=None)
    x = torch.randn(1, 12, 6)
    y = conv(x)
    x2 = x.clone()
    x2[:, 8:] += 1.0
    assert torch.equal(conv(x2)[:, :8], y[:, :8])  # the future does not leak into the past
    cu = torch.tensor([0, 5, 12])
    y_docs = conv(x, cu_seqlens=cu)
    torch.testing.assert_close(y_docs[:, 5:], conv(x[:, 5:]))  # the second document starts from a clean window


def test_gated_delta_rule_chunked_equals_recurrent_and_trains():
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 100, 2, 8, 16
    q, k, v = torch.randn(B, T, H, dk), torch.randn(B, T, H, dk), torch.randn(B, T, H, dv)
    g, beta = -torch.rand(B, T, H), torch.rand(B, T, H) * 2
    torch.testing.assert_close(gated_delta_rule(q, k, v, g, beta, chunk_size=32), gated_delta_rule_recurrent(q, k, v, g, beta),
                               rtol=1e-4, atol=1e-5)
    cfg = GatedDeltaNetConfig(n_heads=2, n_v_heads=4, head_dim=8)
    layer = cfg.build(32)
    layer.init_weights()
    assert sum(p.numel() for p in layer.parameters()) == cfg.num_params(32)
    x = torch.randn(2, 20, 32, requires_grad=True)
    layer(x).sum().backward()
    assert torch.isfinite(x.grad).all()


def test_cross_entropy_module():
    torch.manual_seed(0)
    logits, labels = torch.randn(3, 7, 11), torch.randint(0, 11, (3, 7))
    labels[0, :2] = -100
    ce, z = CrossEntropyLoss(z_loss_multiplier=1e-3)(logits, labels)
    torch.testing.assert_close(ce, F.cross_entropy(logits.view(-1, 11), labels.view(-1), ignore_index=-100))
    mask = labels.view(-1) != -100
    want_z = 1e-3 * (torch.logsumexp(logits.view(-1, 11), -1).pow(2) * mask).sum() / mask.sum()
    torch.testing.assert_close(z, want_z)
    per_token, _ = CrossEntropyLoss(reduction="none")(logits, labels)
    assert per_token.shape == labels.shape and (per_token[0, :2] == 0).all()


def test_fused_linear_cross_entropy_options_match_pytorch():
    import torch
    import torch.nn.functional as F

    from olmo_core_b200.nn.functional import fused_linear_cross_entropy_loss

    torch.manual_seed(0)
    h, w = torch.randn(12, 16), torch.randn(32, 16)
    labels = torch.randint(0, 32, (12,))
    labels[3] = -100
    logits = h @ w.t()
    loss, z = fused_linear_cross_entropy_loss(h, w, labels)
    torch.testing.assert_close(loss, F.cross_entropy(logits, labels, ignore_index=-100))
    assert z is None
    capped = 5.0 * torch.tanh(logits / 5.0)
    loss, _ = fused_linear_cross_entropy_loss(h, w, labels, softcap=5.0)
    torch.testing.assert_close(loss, F.cross_entropy(capped, labels, ignore_index=-100))
    cw = torch.rand(32) + 0.5
    loss, _ = fused_linear_cross_entropy_loss(h, w, labels, ce_weight=cw, label_smoothing=0.1, reduction="sum")
    torch.testing.assert_close(loss, F.cross_entropy(logits, labels, weight=cw, ignore_index=-100, label_smoothing=0.1, reduction="sum"))
    total, z = fused_linear_cross_entropy_loss(h, w, labels, softcap=5.0, compute_z_loss=True, z_loss_multiplier=1e-2)
    keep = labels != -100
    want_z = 1e-2 * (torch.logsumexp(capped, -1).pow(2) * keep).sum() / keep.sum()
    torch.testing.assert_close(z, want_z)
    torch.testing.assert_close(total, F.cross_entropy(capped, labels, ignore_index=-100) + want_z)
