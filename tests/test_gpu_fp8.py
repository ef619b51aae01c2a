"""8-bit floating-point path: quantisation kernels, the e4m3 tcgen05 GEMM and the linear layer built on them."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("pow2", [False, True])
@pytest.mark.parametrize("R,C", [(64, 128), (300, 520), (4096, 1024)])
def test_quantisation_kernels_match_emulation(R, C, pow2):
    from olmo_core_b200.ops.fp8 import quantize_colwise_transposed, quantize_rowwise

    torch.manual_seed(0)
    x = (torch.randn(R, C) * torch.rand(R, 1) * 3).bfloat16()
    for fn in (quantize_rowwise, quantize_colwise_transposed):
        q_ref, s_ref = fn(x, pow2)
        q, s = fn(x.to(DEV), pow2)
        torch.testing.assert_close(s.cpu(), s_ref, rtol=1e-6, atol=0)
        deq = q.cpu().view(torch.float8_e4m3fn).float()
        deq_ref = q_ref.view(torch.float8_e4m3fn).float()
        # identical up to ties of the rounding of x / scale (the division is done as a multiplication on the device)
        assert (deq != deq_ref).float().mean() < 2e-3
        assert _rel_err(deq * s.cpu()[:, None], (x.float() if fn is quantize_rowwise else x.float().t())) < 0.04


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (512, 768, 384), (1000, 520, 272), (4096, 4096, 4096)])
def test_gemm_fp8_matches_dequantised_product(M, N, K):
    from olmo_core_b200.ops import _lib
    from olmo_core_b200.ops.fp8 import gemm_fp8, quantize_rowwise

    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    aq, sa = quantize_rowwise(a)
    bq, sb = quantize_rowwise(b)
    out = gemm_fp8(aq, sa, bq, sb)
    _lib.check_device_status()
    # the tensor cores multiply the e4m3 values exactly and accumulate in fp32: compare with that product in fp32
    ref = (aq.view(torch.float8_e4m3fn).float() @ bq.view(torch.float8_e4m3fn).float().t()) * sa[:, None] * sb[None, :]
    assert _rel_err(out, ref) < 5e-3
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    gemm_fp8(aq, sa, bq, sb, out=acc, accumulate=True)
    assert _rel_err(acc - 1, ref) < 1e-3
    assert _rel_err(out, a.float() @ b.float().t()) < 0.06  # and the quantisation error itself stays at the e4m3 level


@pytest.mark.parametrize("recipe_hp", [False, True])
def test_fp8_linear_autograd(recipe_hp):
    from olmo_core_b200.ops.fp8 import fp8_linear

    torch.manual_seed(2)
    x = torch.randn(4, 256, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(768, 512, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    y = fp8_linear(x, w, pow2_scales=True, wgrad_high_precision=recipe_hp)
    ref = x.float() @ w.float().t()
    assert _rel_err(y, ref) < 0.06
    g = torch.randn_like(y)
    y.backward(g)
    assert _rel_err(x.grad, g.float() @ w.float()) < 0.06
    want_dw = g.float().reshape(-1, 768).t() @ x.float().reshape(-1, 512)
    assert _rel_err(w.grad, want_dw) < (0.01 if recipe_hp else 0.06)


def test_float8_config_routes_projections_through_the_fp8_kernels():
    from olmo_core_b200.float8 import Float8Config
    from olmo_core_b200.nn.transformer import TransformerConfig
    from olmo_core_b200.ops import _lib

    torch.manual_seed(3)
    model = TransformerConfig.olmo2_30M(vocab_size=512, n_layers=2).build(init_device="cpu")
    ref_state = {k: v.clone() for k, v in model.state_dict().items()}
    ids = torch.randint(0, 512, (2, 128), device=DEV)
    model = model.to(DEV, torch.bfloat16)
    base = model(ids).float()
    Float8Config(enabled=True).apply_float8_linear(model)
    marked = [n for n, m in model.named_modules() if getattr(m, "float8", None) is not None]
    assert marked and not any(n.startswith("lm_head") for n in marked)
    before = _lib.launch_count
    out = model(ids).float()
    assert _lib.launch_count > before
    assert _rel_err(out, base) < 0.15 and torch.isfinite(out).all()
    out.sum().backward()
    del ref_state
