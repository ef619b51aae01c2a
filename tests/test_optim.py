"""Optimizers and learning-rate schedules against PyTorch references and closed-form values."""

import math

import pytest
import torch
import torch.nn as nn

from olmo_core_b200.optim import (
    WSD,
    AdamWConfig,
    ConstantWithWarmup,
    CosWithWarmup,
    LinearWithWarmup,
    LionConfig,
    MuonConfig,
    NoOpConfig,
    OptimGroupOverride,
    SchedulerUnits,
    SkipStepAdamWConfig,
)


def _model(seed: int = 0) -> nn.Module:
    torch.manual_seed(seed)
    return nn.Sequential(nn.Embedding(32, 16), nn.Linear(16, 16), nn.Linear(16, 4))


def _step(model, optim, seed):
    torch.manual_seed(seed)
    x = torch.randint(0, 32, (8,))
    loss = model(x).pow(2).mean()
    optim.zero_grad()
    loss.backward()
    optim.step()
    return loss.item()


def test_adamw_matches_torch():
    a, b = _model(), _model()
    ours = AdamWConfig(lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1).build(a)
    ref = torch.optim.AdamW(b.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for s in range(5):
        _step(a, ours, s)
        _step(b, ref, s)
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def test_group_overrides_split_parameters():
    m = _model()
    optim = AdamWConfig(lr=1e-2, weight_decay=0.1,
                        group_overrides=[OptimGroupOverride(params=["0.weight"], opts=dict(weight_decay=0.0))]).build(m)
    decays = sorted(g["weight_decay"] for g in optim.param_groups)
    assert decays == [0.0, 0.1]
    assert sum(len(g["params"]) for g in optim.param_groups) == len(list(m.parameters()))
    with pytest.raises(Exception):
        AdamWConfig(group_overrides=[OptimGroupOverride(params=["missing.*"], opts={})]).build(_model())


def test_skip_step_adamw_skips_outlier_losses():
    a, b = _model(), _model()
    skipper = SkipStepAdamWConfig(lr=1e-2, rolling_interval_length=8, sigma_factor=3).build(a)
    plain = SkipStepAdamWConfig(lr=1e-2, rolling_interval_length=8, sigma_factor=3).build(b)
    for s in range(12):  # identical, well-behaved history
        for model, optim in ((a, skipper), (b, plain)):
            torch.manual_seed(s)
            loss = model(torch.randint(0, 32, (8,))).pow(2).mean()
            optim.zero_grad()
            loss.backward()
            optim.latest_loss = loss.detach()
            optim.latest_grad_norm = torch.tensor(1.0)
            optim.step()
    before = [p.detach().clone() for p in a.parameters()]
    loss = a(torch.randint(0, 32, (8,))).pow(2).mean()
    skipper.zero_grad()
    loss.backward()
    skipper.latest_loss = loss.detach() * 1e6  # a spike far outside the rolling window
    skipper.latest_grad_norm = torch.tensor(1.0)
    skipper.step()
    for p, q in zip(a.parameters(), before):
        torch.testing.assert_close(p, q, rtol=0, atol=0)  # the step was a no-op
    assert float(skipper.step_skipped) == 1.0


def test_lion_update_is_sign_of_interpolated_momentum():
    m = _model()
    optim = LionConfig(lr=1e-3, betas=(0.9, 0.99), weight_decay=0.0).build(m)
    before = [p.detach().clone() for p in m.parameters()]
    _step(m, optim, 0)
    for p, q in zip(m.parameters(), before):
        delta = (p - q).abs()
        touched = delta > 0
        if touched.any():  # first step: momentum is zero, so the update is lr * sign(grad)
            torch.testing.assert_close(delta[touched], torch.full_like(delta[touched], 1e-3), rtol=1e-4, atol=1e-8)


def test_muon_and_noop():
    m = _model()
    optim = MuonConfig(lr=1e-2).build(m)
    losses = [_step(m, optim, 0) for _ in range(20)]
    assert losses[-1] < losses[0]
    n = _model()
    noop = NoOpConfig().build(n)
    before = [p.detach().clone() for p in n.parameters()]
    _step(n, noop, 0)
    for p, q in zip(n.parameters(), before):
        assert torch.equal(p, q)


def test_schedules_closed_form():
    cos = CosWithWarmup(warmup_steps=10, alpha_f=0.1)
    assert float(cos.get_lr(1.0, 0, 100)) == 0.0
    assert float(cos.get_lr(1.0, 5, 100)) == pytest.approx(0.5)
    assert float(cos.get_lr(1.0, 10, 100)) == pytest.approx(1.0)
    mid = 0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 45 / 90))
    assert float(cos.get_lr(1.0, 55, 100)) == pytest.approx(mid)
    assert float(cos.get_lr(1.0, 100, 100)) == pytest.approx(0.1)
    lin = LinearWithWarmup(warmup_steps=10, alpha_f=0.0)
    assert float(lin.get_lr(2.0, 55, 100)) == pytest.approx(1.0)
    const = ConstantWithWarmup(warmup_steps=4)
    assert [float(const.get_lr(1.0, s, 100)) for s in (0, 2, 4, 50)] == pytest.approx([0.0, 0.5, 1.0, 1.0])
    wsd = WSD(warmup_steps=10, decay_steps=20)
    assert float(wsd.get_lr(1.0, 50, 100)) == pytest.approx(1.0)
    assert float(wsd.get_lr(1.0, 90, 100)) == pytest.approx(0.5)
    assert float(wsd.get_lr(1.0, 100, 100)) == pytest.approx(0.0)
    tok = CosWithWarmup(units=SchedulerUnits.tokens, warmup=1000)
    assert float(tok.get_lr(1.0, 500, 10_000)) == pytest.approx(0.5)
